"""A plain, slow Tutezen: whole sequences, no cache, no batching, one function a mechanism.

Tutezen is a decoder whose layers are parallel blocks (one norm; mixer and feed-forward both read its output and
their sum, times a constant, is added to the stream), whose mixers are either a state-space recurrence of the
Mamba-2 kind or attention through low-rank latents with a sliding window, a learned sink per head and an output
gate, whose feed-forwards are a dense GELU layer or a routed mixture of gated experts with a shared one, and in
which a stretch of layers may run several times with the same weights, the embedding output and a learned
vector being added to the stream before each further pass.

Everything here is written from those equations in float64 by default and shares no code with the engine:
configuration is the plain dict of config.json, weights a dict of tensors by name.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def rms_divide(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(z: torch.Tensor) -> torch.Tensor:
    return z / (1.0 + torch.exp(-z))


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def causal_conv(u: torch.Tensor, w: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """u [T, C], w [C, taps], b [C]: out_t = b + sum_j w[:, j] u_(t - taps + 1 + j), zeros before the start."""
    T, C = u.shape
    taps = w.shape[1]
    out = b.expand(T, C).clone()
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                out[t] = out[t] + w[:, j] * u[s]
    return out


def state_space(x, B, C, dt, a_log, d_skip, groups: int):
    """The recurrence head by head.  x [T, heads, P], B and C [T, groups, N], dt [T, heads] (already positive).
    S_t = exp(-exp(a_log) dt_t) S_(t-1) + dt_t B_t x_t^T (N x P); y_t = S_t^T C_t + d_skip x_t."""
    T, H, P = x.shape
    N = B.shape[-1]
    per = H // groups
    y = torch.zeros_like(x)
    for h in range(H):
        g = h // per
        S = torch.zeros(N, P, dtype=x.dtype)
        rate = torch.exp(a_log[h])
        for t in range(T):
            S = torch.exp(-rate * dt[t, h]) * S + dt[t, h] * torch.outer(B[t, g], x[t, h])
            y[t, h] = S.T @ C[t, g] + d_skip[h] * x[t, h]
    return y


def grouped_rms(y: torch.Tensor, parts: int, eps: float) -> torch.Tensor:
    """y [T, n] divided, in ``parts`` equal parts, by each part's own root mean square."""
    T, n = y.shape
    return rms_divide(y.reshape(T, parts, n // parts), eps).reshape(T, n)


def mamba2(h: torch.Tensor, w: Dict[str, torch.Tensor], pre: str, m: dict, eps: float) -> torch.Tensor:
    heads, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = heads * P
    T = h.shape[0]
    proj = h @ w[pre + "in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, w[pre + "conv"], w[pre + "conv.b"]))
    x = xbc[:, :inner].reshape(T, heads, P)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + w[pre + "dt_bias"])
    y = state_space(x, B, C, dt, w[pre + "A_log"], w[pre + "D"], G).reshape(T, inner)
    y = grouped_rms(y * silu(z), m["norm_groups"], eps) * w[pre + "norm"]
    return y @ w[pre + "o"].T


def rotate_pairs(v: torch.Tensor, pos: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """Rotation of the first ``dims`` dimensions of the last axis, dimension 2i with 2i+1, by pos * base^(-2i/dims).
    v [T, ..., d]; pos [T]."""
    out = v.clone()
    i = torch.arange(dims // 2, dtype=v.dtype)
    ang = pos.to(v.dtype)[:, None] * base ** (-2.0 * i / dims)          # [T, dims/2]
    while ang.dim() < v.dim():
        ang = ang.unsqueeze(1)
    cs, sn = torch.cos(ang), torch.sin(ang)
    a, b = v[..., 0:dims:2], v[..., 1:dims:2]
    out[..., 0:dims:2] = a * cs - b * sn
    out[..., 1:dims:2] = b * cs + a * sn
    return out


def windowed_sink_softmax(scores: torch.Tensor, sink: torch.Tensor, window: Optional[int]) -> torch.Tensor:
    """scores [T, T] of one head; row i keeps j with 0 <= i - j < window; the denominator also holds exp(sink)."""
    T = scores.shape[0]
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    keep = (j <= i) & ((i - j < window) if window else torch.ones_like(j, dtype=torch.bool))
    s = torch.where(keep, scores, torch.full_like(scores, -math.inf))
    top = torch.maximum(s.max(-1, keepdim=True).values, sink.reshape(1, 1))
    e = torch.exp(s - top)
    return e / (e.sum(-1, keepdim=True) + torch.exp(sink - top))


def latent_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], pre: str, m: dict, eps: float) -> torch.Tensor:
    H, d, r, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    T = h.shape[0]
    pos = torch.arange(T)
    rot = m.get("rot") or {}
    cq = rms_divide(h @ w[pre + "dq"].T, eps) * w[pre + "dq.norm"]
    q = (cq @ w[pre + "uq"].T).reshape(T, H, d + r)
    kv = h @ w[pre + "dkv"].T
    c = rms_divide(kv[:, :rank], eps) * w[pre + "dkv.norm"]
    k_rot = kv[:, rank:]
    if rot:
        k_rot = rotate_pairs(k_rot, pos, rot["dims"], rot["base"])
        q = torch.cat([q[..., :d], rotate_pairs(q[..., d:], pos, rot["dims"], rot["base"])], -1)
    k = (c @ w[pre + "uk"].T).reshape(T, H, d)
    v = (c @ w[pre + "uv"].T).reshape(T, H, dv)
    window = (m.get("mask") or {}).get("size")
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for a in range(H):
        s = (q[:, a, :d] @ k[:, a].T + q[:, a, d:] @ k_rot.T) * m["scale"]
        out[:, a] = windowed_sink_softmax(s, w[pre + "sink"][a], window) @ v[:, a]
    gate = torch.sigmoid(h @ w[pre + "g"].T)
    return (out.reshape(T, H * dv) * gate) @ w[pre + "o"].T


def dense_ff(h, w, pre):
    return gelu_tanh(h @ w[pre + "up"].T) @ w[pre + "down"].T


def gated_expert(h, w, pre):
    return (silu(h @ w[pre + "gate"].T) * (h @ w[pre + "up"].T)) @ w[pre + "down"].T


def route(h: torch.Tensor, w_router: torch.Tensor, top: int):
    """Chosen experts [T, top] and their weights: softmax over all experts, the top scores divided by their sum."""
    s = torch.softmax(h @ w_router.T, -1)
    val, idx = torch.topk(s, top, dim=-1)
    return idx, val / (val.sum(-1, keepdim=True) + 1e-20)


def moe_ff(h, w, pre, mlp):
    idx, wt = route(h, w[pre + "router"], mlp["router"]["top"])
    out = torch.zeros(h.shape[0], w[pre + "e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for k in range(idx.shape[1]):
            out[t] = out[t] + wt[t, k] * gated_expert(h[t:t + 1], w, f"{pre}e{int(idx[t, k])}.")[0]
    if mlp.get("shared"):
        out = out + gated_expert(h, w, pre + "shared.")
    return out


def layer_order(cfg: dict) -> List[tuple]:
    """(layer, pass number or None, first of its pass) for every layer run."""
    n, loop = len(cfg["layers"]), cfg.get("loop")
    if not loop:
        return [(i, None, False) for i in range(n)]
    runs = [(i, None, False) for i in range(loop["start"])]
    for t in range(loop["times"]):
        runs += [(i, t, i == loop["start"]) for i in range(loop["start"], loop["stop"])]
    return runs + [(i, None, False) for i in range(loop["stop"], n)]


def forward(cfg: dict, weights: Dict[str, torch.Tensor], tokens: List[int], compute=torch.float64, streams: list = None):
    """Logits [T, vocab] of one sequence.  ``streams``: a list that receives the stream after every layer run."""
    w = {k: (v.to(compute) if v.is_floating_point() else v) for k, v in weights.items()}
    eps, mult = cfg["norm"]["eps"], cfg["residual_mult"]
    x0 = w["embed"][torch.tensor(tokens)]
    x = x0.clone()
    for i, t, first in layer_order(cfg):
        if first:
            if t > 0:
                x = x + x0
            x = x + w["loop.step"][t]
        ly, pre = cfg["layers"][i], f"l{i}."
        h = rms_divide(x, eps) * w[pre + "norm1"]
        if ly["type"] == "mamba2":
            a = mamba2(h, w, pre + "mix.", ly["mixer"], eps)
        elif ly["type"] == "latent_attention":
            a = latent_attention(h, w, pre + "mix.", ly["mixer"], eps)
        else:
            raise ValueError(ly["type"])
        mlp = ly.get("mlp")
        if mlp is not None:
            a = a + (dense_ff(h, w, pre + "mlp.") if mlp["kind"] == "dense" else moe_ff(h, w, pre + "mlp.", mlp))
        x = x + mult * a
        if streams is not None:
            streams.append(x.clone())
    return (rms_divide(x, eps) * w["final.norm"]) @ w["embed"].T
