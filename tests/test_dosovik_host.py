"""Dosovik through the engine's host side without a GPU: configuration, weights by name, the block's
arrangement, the convolution state by slot, value mixing between layers, pages and slots used again, the
scheduler.  The kernels are the torch stand-ins of host_ops.py; what the CUDA kernels compute is tested on the GPU."""
import io
import json

import numpy as np
import pytest
import torch

import dosovik_helpers as DH
import helpers
from host_ops import HostOps


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for i, name in enumerate(DH.CONFIGS):
        d = str(tmp_path_factory.mktemp("dosovik" + name))
        DH.make_model(d, name, seed=10 + i)
        out[name] = (d,) + DH.CONFIGS[name]
    return out


def _replay(d, steps, out_dir, max_tokens, page):
    from atoma_infer_b200.engine.trace import replay

    steps = helpers.number(steps)
    text = "\n".join(json.dumps(s) for s in steps) + "\n"
    replay(d, "float32", out_dir, max_tokens, stream=io.StringIO(text), out=io.StringIO(), page_size=page, device="cpu",
           ops=HostOps())
    return steps


@pytest.mark.parametrize("name", list(DH.CONFIGS))
def test_every_cutting_matches_plain(name, models, tmp_path):
    d, cfg, page = models[name]
    seqs = helpers.random_tokens(cfg["vocab"], (1, 2, 9, 30, 47), seed=5)
    ref = DH.plain_logits(d, cfg, seqs)
    steps = (helpers.trace_whole(seqs) + helpers.trace_tail(seqs, tail=12) + helpers.trace_chunks(seqs, sizes=(5, 2, 7, 3, 2, 11, 1, 4))
             + helpers.trace_mixed(seqs, sizes=(6, 2, 9, 3, 5)))
    steps = _replay(d, steps, str(tmp_path), 192, page)  # four live requests at most, 64 tokens each: pages come back
    worst, where, agree, _ = helpers.compare_trace(steps, str(tmp_path), cfg["vocab"], ref)
    assert worst <= helpers.FP32_TOL, (worst, where)
    assert agree == 1.0


def test_config_is_read_key_by_key(models):
    from atoma_infer_b200.config import ConfigError
    from atoma_infer_b200.config.dosovik_config import DosovikConfig

    cfg = DH.CONFIGS["Q"][0]
    c = DosovikConfig.from_dict(cfg)
    assert (c.width, c.vocab, c.taps, c.alpha) == (128, 300, 5, 1.5)
    assert c.layers[1].mlp is None and c.layers[0].mlp.ff == 192
    assert (c.layers[0].mixer.dim, c.layers[0].mixer.vdim, c.layers[0].mixer.chunk) == (16, 32, 40)
    bad = json.loads(json.dumps(cfg))
    bad["layers"][0]["type"] = "recurrent"
    with pytest.raises(ConfigError, match="recurrent"):
        DosovikConfig.from_dict(bad)
    bad = json.loads(json.dumps(cfg))
    del bad["layers"][2]["mixer"]["vdim"]
    with pytest.raises(ConfigError, match="vdim"):
        DosovikConfig.from_dict(bad)


def test_a_missing_tensor_is_named(models, tmp_path):
    from atoma_infer_b200.engine.runtime import load_model
    from atoma_infer_b200.weights.loader import WeightError
    from atoma_infer_b200.weights.safetensors_io import write_safetensors

    d, cfg, page = models["P"]
    w = {k: v.to(torch.bfloat16) for k, v in helpers.read_weights(d).items() if k != "l1.mix.k.norm"}
    with open(tmp_path / "config.json", "w") as f:
        json.dump(cfg, f)
    write_safetensors(str(tmp_path / "model.safetensors"), w, {})
    with pytest.raises(WeightError, match="l1.mix.k.norm"):
        load_model(str(tmp_path), dtype="float32", device="cpu", ops=HostOps(), num_pages=8, page_size=page, max_seqs=2)


def test_greedy_generation_through_the_scheduler(models):
    """Few pages and a small token budget: prompts are cut, requests preempted and recomputed, slots used again."""
    from atoma_infer_b200.engine import Engine
    from atoma_infer_b200.sampling import SamplingParams

    d, cfg, page = models["P"]
    prompts = list(helpers.random_tokens(cfg["vocab"], (3, 26, 9, 17, 5), seed=8).values())
    want = [DH.plain_greedy(d, cfg, p, 10) for p in prompts]
    eng = Engine(d, dtype="float32", block_size=page, cuda_graphs=False, ops=HostOps(), num_gpu_blocks_override=22,
                 max_num_sequences=3, max_num_batched_tokens=11)
    outs = eng.generate(prompts, SamplingParams(do_sample=False, max_new_tokens=10, ignore_eos_token=True))
    assert [o.token_ids for o in outs] == want
    assert eng.lm.manager.audit() == "" and eng.lm.manager.num_requests() == 0
