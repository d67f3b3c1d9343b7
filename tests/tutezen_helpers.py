"""Small Tutezen configurations for the tests, their model folders, and the plain logits of token lists.

The configurations differ in every size and constant, and pick values that make mechanisms distinguishable: state
sizes that are no multiple of 16 and one that two threads share, one group of B and C for all heads and several, two
to five taps, the gated norm in one part and in several, windows that are no multiple of a page (and one that is,
and none), a rotation over part of the rotated dimensions, more heads than one tile of the tensor-core kernels
takes, one chosen expert and several, with and without a shared expert, layers without a feed-forward, a stretch of
layers that runs twice or three times, from the first layer on or later, and no repetition at all.
"""
from __future__ import annotations

from typing import Dict, List

import torch

import helpers
import plain_tutezen as PT


def mamba(heads, vdim, state, groups, conv, norm_groups, mlp=None):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv,
                                        "norm_groups": norm_groups}, "mlp": mlp}


def latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, window=None, rot_dims=None, base=10000.0, mlp=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": scale}
    if window:
        m["mask"] = {"size": window}
    if rot_dims:
        m["rot"] = {"dims": rot_dims, "base": base}
    return {"type": "latent_attention", "mixer": m, "mlp": mlp}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, shared=0):
    m = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def config(width, vocab, layers, mult, loop=None, eps=1e-5):
    c = {"architecture": "Tutezen", "vocab": vocab, "width": width, "norm": {"eps": eps}, "residual_mult": mult, "layers": layers}
    if loop:
        c["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return c


# name -> (config, page size)
CONFIGS = {
    # the first two layers run three times; a state of 24 rows, a window of 21 keys over pages of 4, values larger
    # than keys, a layer without feed-forward
    "P": (config(96, 131, [mamba(3, 16, 24, 1, 4, 3, dense(160)),
                           latent(3, 16, 8, 24, 40, 48, 0.2, window=21, rot_dims=8, mlp=moe(5, 2, 48, shared=64)),
                           mamba(4, 8, 40, 2, 2, 1)], mult=0.7, loop=(0, 2, 3)), 4),
    # no repetition; twenty heads (the plain attention kernel in both modes), no window, a rotation over half of the rotated
    # dimensions; one chosen expert, no shared one; factor 1
    "Q": (config(128, 300, [latent(20, 8, 16, 8, 24, 32, 0.3, rot_dims=8, base=5e5, mlp=dense(192)),
                            mamba(2, 64, 16, 2, 3, 2, moe(4, 1, 32))], mult=1.0, eps=1e-6), 16),
    # the second layer alone runs twice; a state of 128 rows (two threads a column), four groups, five taps; a cached
    # vector of 112 elements, a window of 64 keys = 8 pages, no rotation at all; three chosen experts of eight
    "R": (config(64, 97, [mamba(8, 8, 128, 4, 5, 4, moe(8, 3, 16, shared=32)),
                          latent(2, 32, 16, 16, 16, 96, 0.125, window=64),
                          latent(4, 16, 16, 16, 32, 48, 0.25, window=9, rot_dims=16, mlp=dense(80))], mult=0.5, loop=(1, 2, 2)), 8),
}

# stds that make every mechanism matter: sinks of order one, a decisive router, step sizes that differ from head to head
# (short and long memories), convolutions and the vectors added between passes far from zero
SCALES = {"sink": 30.0, "router": 8.0, "dt_bias": 40.0, "A_log": 10.0, "conv": 6.0, "loop.step": 10.0}


def make_model(path: str, name: str, seed: int = 0) -> str:
    cfg, _ = CONFIGS[name]
    return helpers.make_model(path, cfg, seed=seed, scales=SCALES, norm_jitter=0.2)


def plain_logits(model_dir: str, cfg: dict, seqs: Dict[str, List[int]]) -> Dict[str, torch.Tensor]:
    w = helpers.read_weights(model_dir)
    return {k: PT.forward(cfg, w, v) for k, v in seqs.items()}


def plain_greedy(model_dir: str, cfg: dict, prompt: List[int], n: int) -> List[int]:
    w = helpers.read_weights(model_dir)
    toks, out = list(prompt), []
    for _ in range(n):
        t = int(torch.argmax(PT.forward(cfg, w, toks)[-1]))
        out.append(t)
        toks.append(t)
    return out
