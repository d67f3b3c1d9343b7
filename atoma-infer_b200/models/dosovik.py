"""Dosovik as a model spec: post-norm blocks whose sublayers read the stream through a short convolution,
attention with biases, whole-projection query/key norms, a partial rotation, a chunk mask, a softmax sink and
value mixing, and a dense feed-forward with the polynomial activation of normalised powers.

Tensor names: ``embed``, ``head``, ``final.norm``; layer i under ``l<i>.``: ``norm1``, ``norm2``, ``canon1``,
``canon2``, ``mix.{q,k,v,o}``, ``mix.{q,k,v}.b``, ``mix.{q,k}.norm``, ``mix.vmix``, ``mlp.{up,down,act}``.
"""
from __future__ import annotations

from ..config.dosovik_config import DosovikConfig
from ..config.registry import register_architecture
from ..parts.model import LayerSpec, ModelSpec

_ATTENTION_NAMES = {"q": ".q", "k": ".k", "v": ".v", "o": ".o", "q_bias": ".q.b", "k_bias": ".k.b", "v_bias": ".v.b",
                    "q_norm": ".q.norm", "k_norm": ".k.norm", "v_mix": ".vmix"}


def dosovik_spec(cfg: DosovikConfig) -> ModelSpec:
    # norm weights are stored around zero: the factor is 1 + w
    norm = {"kind": "rmsnorm", "size": cfg.width, "eps": cfg.eps, "weight_offset": 1.0, "tensor_suffix": ""}
    flt = {"kind": "short_conv", "channels": cfg.width, "taps": cfg.taps} if cfg.taps else None
    layers, ignored = [], []
    for i, ly in enumerate(cfg.layers):
        a = ly.mixer
        position = ({"kind": "rope", "head_dim": a.dim, "rotary_dim": a.rot_dims, "theta": a.rot_base, "exact_frequencies": True}
                    if a.rot_dims else {"kind": "none", "head_dim": a.dim})
        mixer = {
            "kind": "attention", "hidden": cfg.width, "num_heads": a.heads, "num_kv_heads": a.kv_heads, "head_dim": a.dim,
            "v_head_dim": a.vdim, "scale": a.scale, "window": None, "chunk": a.chunk, "sink": True, "bias": True,
            "qk_norm": {"eps": cfg.eps}, "v_mix": {"key": "first"} if a.v_mix else None, "position": position,
            "names": _ATTENTION_NAMES,
        }
        ff = ({"kind": "polynorm", "hidden": cfg.width, "intermediate": ly.mlp.ff, "eps": cfg.eps} if ly.mlp else None)
        layers.append(LayerSpec(f"l{i}", {"kind": "postnorm", "norm": norm, "mixer": mixer, "feed_forward": ff,
                                          "alpha": cfg.alpha, "filter": flt}))
        if not a.v_mix:
            ignored.append(f"l{i}.mix.vmix")
        if ly.mlp is None:  # a layer without a feed-forward has no second sum
            ignored += [f"l{i}.norm2", f"l{i}.canon2"]
    return ModelSpec(
        hidden_size=cfg.width, vocab_size=cfg.vocab, layers=layers, final_norm=norm, final_norm_prefix="final.norm",
        embedding={"kind": "token", "vocab": cfg.vocab, "hidden": cfg.width, "tensor": "embed", "scale": cfg.embedding_scale},
        head={"kind": "linear", "vocab": cfg.vocab, "hidden": cfg.width, "tensor": "head"},
        ignored_tensors=tuple(ignored),
    )


register_architecture("Dosovik", DosovikConfig.from_dict, dosovik_spec, model_type="dosovik")
