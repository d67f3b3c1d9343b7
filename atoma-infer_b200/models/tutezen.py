"""Tutezen as a model spec: parallel blocks (one norm, mixer and feed-forward side by side, their sum times a constant
added to the stream) whose mixers are Mamba-2 state-space layers or latent attention with a sliding window, a learned
sink per head and an output gate, and whose feed-forwards are a dense GELU layer or routed experts with a shared one.
A stretch of layers may run several times in a row with the same weights: every pass is a run of the schedule
with a cache and a state of its own, and before each pass the stream receives the embedding output (not before the
first pass) and that pass's row of a learned table.  The head is the embedding matrix.

Tensor names: ``embed``, ``final.norm``, ``loop.step``; layer i under ``l<i>.``: ``norm1``; Mamba-2 ``mix.{in,conv,
conv.b,dt_bias,A_log,D,norm,o}``; latent attention ``mix.{dq,dq.norm,uq,dkv,dkv.norm,uk,uv,sink,g,o}``; dense
feed-forward ``mlp.{up,down}``; experts ``mlp.router``, ``mlp.e<j>.{gate,up,down}``, ``mlp.shared.{gate,up,down}``.
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.tutezen_config import DenseFF, LatentAttentionSizes, Mamba2Sizes, MoEFF, TutezenConfig
from ..parts.model import LayerRun, LayerSpec, ModelSpec, StreamAdd


def _mixer(cfg: TutezenConfig, m):
    if isinstance(m, Mamba2Sizes):
        return {"kind": "mamba2", "hidden": cfg.width, "heads": m.heads, "head_dim": m.vdim, "state": m.state,
                "groups": m.groups, "taps": m.conv, "norm_groups": m.norm_groups, "eps": cfg.eps}
    assert isinstance(m, LatentAttentionSizes)
    return {"kind": "latent_attention", "hidden": cfg.width, "heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim,
            "v_head_dim": m.vdim, "q_rank": m.q_rank, "kv_rank": m.kv_rank, "scale": m.scale, "window": m.window,
            "rotary_dims": m.rot_dims, "theta": m.rot_base, "eps": cfg.eps, "sink": True, "gate": True}


def _feed_forward(cfg: TutezenConfig, f):
    if f is None:
        return None
    if isinstance(f, DenseFF):
        return {"kind": "dense_act", "hidden": cfg.width, "intermediate": f.ff, "activation": "gelu_tanh"}
    assert isinstance(f, MoEFF)
    return {"kind": "routed_experts", "hidden": cfg.width, "experts": f.experts, "top": f.top,
            "intermediate": f.expert_ff, "shared_intermediate": f.shared_ff}


def tutezen_spec(cfg: TutezenConfig) -> ModelSpec:
    norm = {"kind": "rmsnorm", "size": cfg.width, "eps": cfg.eps, "tensor_suffix": ""}
    layers = [LayerSpec(f"l{i}", {"kind": "parallel", "norm": norm, "mixer": _mixer(cfg, ly.mixer),
                                  "feed_forward": _feed_forward(cfg, ly.mlp), "mult": cfg.residual_mult})
              for i, ly in enumerate(cfg.layers)]
    n, loop = len(layers), cfg.loop
    tables = {}
    if loop is None:
        schedule = None
    else:
        tables["loop.step"] = (loop.times, cfg.width)
        schedule = [LayerRun(i) for i in range(loop.start)]
        for t in range(loop.times):
            for i in range(loop.start, loop.stop):
                first = i == loop.start
                schedule.append(LayerRun(i, before=StreamAdd(embedding=t > 0, table="loop.step", row=t) if first else None))
        schedule += [LayerRun(i) for i in range(loop.stop, n)]
    return ModelSpec(
        hidden_size=cfg.width, vocab_size=cfg.vocab, layers=layers, final_norm=norm, final_norm_prefix="final.norm",
        embedding={"kind": "token", "vocab": cfg.vocab, "hidden": cfg.width, "tensor": "embed"},
        head={"kind": "linear", "vocab": cfg.vocab, "hidden": cfg.width, "tensor": None},
        schedule=schedule, stream_tables=tables,
    )


register_architecture("Tutezen", TutezenConfig.from_dict, tutezen_spec, model_type="tutezen")
