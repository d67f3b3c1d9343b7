"""Tutezen through the engine's host side without a GPU: configuration, weights by name, the parallel block and its
pending sum, layers that run several times with a cache and a state of their own, what the stream receives before a
pass, the recurrence's state and the convolution's ring by slot, windows whose pages go back, the scheduler.  The
kernels are the torch stand-ins of host_ops.py; what the CUDA kernels compute is tested on the GPU."""
import io
import json

import pytest
import torch

import helpers
import tutezen_helpers as TH
from host_ops import HostOps


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for i, name in enumerate(TH.CONFIGS):
        d = str(tmp_path_factory.mktemp("tutezen" + name))
        TH.make_model(d, name, seed=30 + i)
        out[name] = (d,) + TH.CONFIGS[name]
    return out


def _replay(d, steps, out_dir, max_tokens, page):
    from atoma_infer_b200.engine.trace import replay

    steps = helpers.number(steps)
    text = "\n".join(json.dumps(s) for s in steps) + "\n"
    replay(d, "float32", out_dir, max_tokens, stream=io.StringIO(text), out=io.StringIO(), page_size=page, device="cpu",
           ops=HostOps())
    return steps


@pytest.mark.parametrize("name", list(TH.CONFIGS))
def test_every_cutting_matches_plain(name, models, tmp_path):
    d, cfg, page = models[name]
    seqs = helpers.random_tokens(cfg["vocab"], (1, 2, 9, 30, 47), seed=5)
    ref = TH.plain_logits(d, cfg, seqs)
    steps = (helpers.trace_whole(seqs) + helpers.trace_tail(seqs, tail=12) + helpers.trace_chunks(seqs, sizes=(5, 2, 7, 3, 2, 11, 1, 4))
             + helpers.trace_mixed(seqs, sizes=(6, 2, 9, 3, 5)))
    steps = _replay(d, steps, str(tmp_path), 192, page)  # four live requests at most, 64 tokens each: pages come back
    worst, where, agree, _ = helpers.compare_trace(steps, str(tmp_path), cfg["vocab"], ref)
    assert worst <= helpers.FP32_TOL, (worst, where)
    assert agree == 1.0


def test_the_stream_after_every_layer_run(models):
    """The stream with its pending sum after every run of the schedule against the plain implementation's: a layer that
    runs again counts each time, and what a pass receives at its start shows in its first run."""
    import numpy as np

    from atoma_infer_b200.engine.runtime import load_model
    from atoma_infer_b200.engine.step import StepEntry
    from atoma_infer_b200.parts.base import PendingSum

    d, cfg, page = models["P"]
    toks = helpers.random_tokens(cfg["vocab"], (19,), seed=2)["r0"]
    want = []
    import plain_tutezen as PT
    PT.forward(cfg, helpers.read_weights(d), toks, streams=want)
    lm = load_model(d, dtype="float32", device="cpu", ops=HostOps(), num_pages=16, page_size=page, max_seqs=2)
    got = []

    def watch(run, resid, delta):
        x = resid.clone()
        assert isinstance(delta, PendingSum) and delta.rows is None and delta.vector is None
        for t in delta.terms:
            x += delta.mult * t.float()
        got.append(x)

    lm.model.watch = watch
    lm.step.run([StepEntry(0, toks, [len(toks) - 1])])
    assert len(got) == len(want) == 3 * 2 + 1
    for a, b in zip(got, want):
        assert float((a.double() - b).abs().max()) < 1e-4 * float(b.abs().max())


def test_config_is_read_key_by_key():
    from atoma_infer_b200.config import ConfigError
    from atoma_infer_b200.config.tutezen_config import TutezenConfig

    cfg = TH.CONFIGS["P"][0]
    c = TutezenConfig.from_dict(cfg)
    assert (c.width, c.vocab, c.residual_mult, c.eps) == (96, 131, 0.7, 1e-5)
    assert (c.loop.start, c.loop.stop, c.loop.times) == (0, 2, 3)
    assert (c.layers[0].mixer.state, c.layers[0].mixer.conv, c.layers[0].mixer.norm_groups) == (24, 4, 3)
    assert (c.layers[1].mixer.kv_rank, c.layers[1].mixer.window, c.layers[1].mixer.rot_dims) == (48, 21, 8)
    assert (c.layers[1].mlp.experts, c.layers[1].mlp.top, c.layers[1].mlp.shared_ff) == (5, 2, 64) and c.layers[2].mlp is None
    assert TutezenConfig.from_dict(TH.CONFIGS["Q"][0]).loop is None
    for path, value, word in ((("layers", 0, "type"), "rwkv", "rwkv"), (("layers", 1, "mlp", "kind"), "sparse", "sparse"),
                              (("layers", 1, "mixer", "kv_rank"), None, "kv_rank"), (("loop", "stop"), 7, "loop"),
                              (("layers", 0, "mixer", "groups"), 2, "groups"), (("layers", 1, "mlp", "router", "top"), 6, "top")):
        bad = json.loads(json.dumps(cfg))
        at = bad
        for key in path[:-1]:
            at = at[key]
        if value is None:
            del at[path[-1]]
        else:
            at[path[-1]] = value
        with pytest.raises(ConfigError, match=word):
            TutezenConfig.from_dict(bad)


def test_the_schedule_gives_every_pass_a_cache_and_a_state_of_its_own():
    from atoma_infer_b200.config.tutezen_config import TutezenConfig
    from atoma_infer_b200.models.tutezen import tutezen_spec
    from atoma_infer_b200.parts.model import DecoderModel

    m = DecoderModel(tutezen_spec(TutezenConfig.from_dict(TH.CONFIGS["P"][0])))
    assert [r.layer for r in m.runs] == [0, 1, 0, 1, 0, 1, 2]
    assert [(r.before.embedding, r.before.row) if r.before else None for r in m.runs] == [(False, 0), None, (True, 1), None,
                                                                                           (True, 2), None, None]
    assert m.run_owner == list(range(7))                      # no run reads another's cache
    assert len(m.groups) == 1 and m.groups[0].layers == [1, 3, 5] and m.groups[0].need.window == 21
    assert [b > 0 for b in m.state_bytes] == [True, False, True, False, True, False, True]
    m = DecoderModel(tutezen_spec(TutezenConfig.from_dict(TH.CONFIGS["R"][0])))
    assert [r.layer for r in m.runs] == [0, 1, 1, 2] and len(m.groups) == 2  # windows of 64 and of 9: pools of their own


def test_a_missing_tensor_is_named(models, tmp_path):
    from atoma_infer_b200.engine.runtime import load_model
    from atoma_infer_b200.weights.loader import WeightError
    from atoma_infer_b200.weights.safetensors_io import write_safetensors

    d, cfg, page = models["P"]
    w = {k: v.to(torch.bfloat16) for k, v in helpers.read_weights(d).items() if k not in ("l1.mix.sink", "loop.step")}
    with open(tmp_path / "config.json", "w") as f:
        json.dump(cfg, f)
    write_safetensors(str(tmp_path / "model.safetensors"), w, {})
    with pytest.raises(WeightError, match="l1.mix.sink") as err:
        load_model(str(tmp_path), dtype="float32", device="cpu", ops=HostOps(), num_pages=8, page_size=page, max_seqs=2)
    assert "loop.step" in str(err.value)


def test_greedy_generation_through_the_scheduler(models):
    """Few pages and a small token budget: prompts are cut, requests preempted and recomputed, slots used again."""
    from atoma_infer_b200.engine import Engine
    from atoma_infer_b200.sampling import SamplingParams

    d, cfg, page = models["P"]
    prompts = list(helpers.random_tokens(cfg["vocab"], (3, 26, 9, 17, 5), seed=8).values())
    want = [TH.plain_greedy(d, cfg, p, 10) for p in prompts]
    eng = Engine(d, dtype="float32", block_size=page, cuda_graphs=False, ops=HostOps(), num_gpu_blocks_override=22,
                 max_num_sequences=3, max_num_batched_tokens=11)
    outs = eng.generate(prompts, SamplingParams(do_sample=False, max_new_tokens=10, ignore_eos_token=True))
    assert [o.token_ids for o in outs] == want
    assert eng.lm.manager.audit() == "" and eng.lm.manager.num_requests() == 0
