"""Small Dosovik configurations for the tests, their model folders, and the plain logits of token lists.

The configurations differ in every size and constant, and pick values that make mechanisms distinguishable:
query/key and value heads of different and of equal size, a rotation over part of a head and over all of it,
two, three and five taps, chunks that are no multiple of a page (and one that is), layers with and without value
mixing, a layer without feed-forward, one key/value head per query head and one for all, alpha other than 1.
"""
from __future__ import annotations

import math
from typing import Dict, List

import torch

import helpers
import plain_dosovik as PD


def _layer(heads, kv, dim, vdim, chunk, rot_dims, base, v_mix, ff, scale=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else 1 / math.sqrt(dim),
         "v_mix": v_mix}
    if chunk:
        m["mask"] = {"size": chunk}
    if rot_dims:
        m["rot"] = {"dims": rot_dims, "base": base}
    return {"type": "attention", "mixer": m, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def config(width, vocab, layers, taps, alpha, eps=1e-5, emb_scale=None):
    c = {"architecture": "Dosovik", "vocab": vocab, "width": width, "norm": {"eps": eps}, "postln_alpha": alpha,
         "embedding": {"scale": emb_scale if emb_scale is not None else math.sqrt(width)}, "layers": layers}
    if taps:
        c["canon"] = {"taps": taps}
    return c


# name -> (config, page size)
CONFIGS = {
    # values smaller than keys, rotation over a third of the head, chunk 21 (pages of 4), three taps,
    # the middle layer takes no part in the value mixing
    "P": (config(96, 131, [_layer(6, 2, 24, 16, 21, 8, 1e4, True, 160), _layer(6, 2, 24, 16, 21, 8, 1e4, False, 160),
                           _layer(6, 2, 24, 16, 21, 8, 1e4, True, 200)], taps=3, alpha=2.0), 4),
    # values larger than keys, every head its own key/value head, rotation over the whole head, chunk 40 (pages of 16),
    # five taps, the second layer has no feed-forward
    "Q": (config(128, 300, [_layer(4, 4, 16, 32, 40, 16, 5e5, True, 192), _layer(4, 4, 16, 32, 40, 16, 5e5, True, 0),
                            _layer(4, 4, 16, 32, 40, 16, 5e5, True, 192)], taps=5, alpha=1.5, eps=1e-6), 16),
    # equal sizes of 64 (no padding; the size of the larger tensor-core kernels), one key/value head for all, chunk 64
    # = 8 pages, two taps, layers that differ from one another in heads and chunk
    "R": (config(256, 512, [_layer(4, 1, 64, 64, 64, 32, 1e6, True, 384), _layer(2, 1, 64, 64, 96, 64, 1e4, True, 256)],
                 taps=2, alpha=4.0, emb_scale=3.0), 8),
    # no convolution, no chunk, no rotation in the second layer, alpha 1: every option off once
    "S": (config(64, 97, [_layer(2, 1, 32, 32, 0, 16, 1e4, False, 96), _layer(2, 2, 32, 32, 0, 0, 1.0, False, 96)],
                 taps=0, alpha=1.0), 8),
}

# stds that make every mechanism matter: biases and the mixing scalar far from zero, activation coefficients of order one
SCALES = {".b": 6.0, "vmix": 8.0, ".act": 12.0, "canon": 6.0}


def make_model(path: str, name: str, seed: int = 0) -> str:
    cfg, _ = CONFIGS[name]
    return helpers.make_model(path, cfg, seed=seed, scales=SCALES, norm_jitter=0.2)


def plain_logits(model_dir: str, cfg: dict, seqs: Dict[str, List[int]]) -> Dict[str, torch.Tensor]:
    w = helpers.read_weights(model_dir)
    return {k: PD.forward(cfg, w, v) for k, v in seqs.items()}


def plain_greedy(model_dir: str, cfg: dict, prompt: List[int], n: int) -> List[int]:
    w = helpers.read_weights(model_dir)
    toks, out = list(prompt), []
    for _ in range(n):
        t = int(torch.argmax(PD.forward(cfg, w, toks)[-1]))
        out.append(t)
        toks.append(t)
    return out
