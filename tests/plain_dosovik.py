"""A plain, slow Dosovik: whole sequences, no cache, no batching, one function a mechanism.

Dosovik is a decoder whose layers normalise AFTER the sum (x <- norm(alpha x + sublayer(x))), whose sublayers
read their input through a short causal convolution over time, whose attention adds biases, normalises the whole
query and key projections, rotates part of each head, looks only inside fixed chunks of positions, has a sink in
its softmax and mixes the values of the first such layer into later ones, and whose feed-forward uses a
polynomial activation of normalised powers.

Everything here is written from those equations in the dtype of ``compute`` (float64 by default) and shares no
code with the engine: configuration is the plain dict of config.json, weights a dict of tensors by name.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def rms_divide(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def one_plus_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """The layer norm of the design: weights are stored around zero."""
    return rms_divide(x, eps) * (1.0 + w)


def short_conv(h: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """Causal convolution over time on each channel: h [T, C], w [C, taps]; out_t = sum_j w[:, j] h_(t-taps+1+j),
    zeros before the start."""
    T, C = h.shape
    taps = w.shape[1]
    out = torch.zeros_like(h)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                out[t] += w[:, j] * h[s]
    return out


def partial_rotation(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x [T, heads, d]: the first ``dims`` of each head rotate, dimension i with i + dims/2, by angle
    position * base^(-2i/dims); the rest pass."""
    half = dims // 2
    out = x.clone()
    for i in range(half):
        f = float(base) ** (-2.0 * i / dims)
        a = positions.to(x.dtype) * f
        c, s = torch.cos(a)[:, None], torch.sin(a)[:, None]
        u, v = x[..., i], x[..., i + half]
        out[..., i] = u * c - v * s
        out[..., i + half] = v * c + u * s
    return out


def chunk_sink_attention(q, k, v, scale: float, chunk: Optional[int], rows=None) -> torch.Tensor:
    """q [T, H, d], k [T, G, d], v [T, G, dv].  Position i sees j <= i of its own chunk (all j <= i without one);
    weights exp(s_j) / (1 + sum exp(s_j)).  ``rows``: the positions to compute (the others stay zero)."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        for i in (range(T) if rows is None else rows):
            lo = (i // chunk) * chunk if chunk else 0
            s = (k[lo:i + 1, g] @ q[i, h]) * scale
            m = max(float(s.max()), 0.0)
            e = torch.exp(s - m)
            p = e / (math.exp(-m) + e.sum())
            out[i, h] = p @ v[lo:i + 1, g]
    return out


def attention_mixer(h: torch.Tensor, positions: torch.Tensor, mx: dict, w: Dict[str, torch.Tensor], pre: str, eps: float,
                    v_first: Optional[torch.Tensor]):
    """Returns (output [T, width], the values this layer cached [T, G, dv])."""
    H, G, d, dv = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    T = h.shape[0]
    q = h @ w[pre + ".q"].T + w[pre + ".q.b"]
    k = h @ w[pre + ".k"].T + w[pre + ".k.b"]
    v = h @ w[pre + ".v"].T + w[pre + ".v.b"]
    q = rms_divide(q, eps) * w[pre + ".q.norm"]
    k = rms_divide(k, eps) * w[pre + ".k.norm"]
    rot = mx.get("rot")
    q, k, v = q.view(T, H, d), k.view(T, G, d), v.view(T, G, dv)
    if rot:
        q = partial_rotation(q, positions, rot["dims"], rot["base"])
        k = partial_rotation(k, positions, rot["dims"], rot["base"])
    if mx.get("v_mix") and v_first is not None:
        lam = w[pre + ".vmix"]
        v = (1.0 - lam) * v + lam * v_first
    mask = mx.get("mask") or {}
    o = chunk_sink_attention(q, k, v, mx["scale"], mask.get("size"))
    return o.reshape(T, H * dv) @ w[pre + ".o"].T, v


def poly_norm(z: torch.Tensor, act: torch.Tensor, eps: float) -> torch.Tensor:
    a, b, c, e = act[0], act[1], act[2], act[3]
    return a * rms_divide(z, eps) + b * rms_divide(z * z, eps) + c * rms_divide(z * z * z, eps) + e


def dense_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], pre: str, eps: float) -> torch.Tensor:
    return poly_norm(h @ w[pre + ".up"].T, w[pre + ".act"], eps) @ w[pre + ".down"].T


def forward(cfg: dict, weights: Dict[str, torch.Tensor], tokens: List[int], compute=torch.float64, layers_out=None):
    """Logits [T, vocab] of one whole sequence.  ``layers_out``: a list that gets the stream after every layer."""
    w = {n: t.to(compute) for n, t in weights.items()}
    eps, alpha = cfg["norm"]["eps"], cfg["postln_alpha"]
    pos = torch.arange(len(tokens))
    x = w["embed"][torch.tensor(tokens)] * cfg["embedding"]["scale"]
    v_first = None
    for i, ly in enumerate(cfg["layers"]):
        pre = f"l{i}"
        assert ly["type"] == "attention"
        h = x + short_conv(x, w[pre + ".canon1"]) if cfg.get("canon") else x
        m, v = attention_mixer(h, pos, ly["mixer"], w, pre + ".mix", eps, v_first)
        if ly["mixer"].get("v_mix") and v_first is None:
            v_first = v
        x = one_plus_norm(alpha * x + m, w[pre + ".norm1"], eps)
        if ly.get("mlp"):
            h = x + short_conv(x, w[pre + ".canon2"]) if cfg.get("canon") else x
            x = one_plus_norm(alpha * x + dense_ff(h, w, pre + ".mlp", eps), w[pre + ".norm2"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    x = one_plus_norm(x, w["final.norm"], eps)
    return x @ w["head"].T
