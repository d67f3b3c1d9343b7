"""Attention through low-rank latents: queries, keys and values are projected up from small vectors, and only the
key/value latent and one rotated key part are cached per token.

With H heads of ``dim`` unrotated and ``rot_dim`` rotated query/key dimensions and ``v_head_dim`` values:
c_q = rmsnorm(W_dq h) (weight, eps), q = W_uq c_q, head by head [dim | rot_dim].  W_dkv h has kv_rank + rot_dim rows:
c = rmsnorm(first kv_rank) is the latent, the last rot_dim rows are a key part shared by all heads.  The rotated
parts of q and k turn by position: of their first ``rotary_dims`` dimensions, 2i pairs with 2i+1, angle
pos * theta^(-2i / rotary_dims).  Per head k = W_uk c and v = W_uv c; score = (q_unrotated . k + q_rotated .
k_rotated) * scale over the keys inside the sliding window; the softmax's denominator also holds exp(sink_h), a
learned number per head without key or value; the heads' outputs, concatenated, are multiplied by sigmoid(W_g h)
and projected out.

How it runs: W_uk is moved onto the query (q' = W_uk,h^T q_unrotated, so that q' . c = q_unrotated . k) and W_uv
behind the attention (o_h = W_uv,h sum_j p_j c_j), which makes it attention of H query heads over ONE key/value head
whose key and value are the same cached vector [c | rotated key part], of size kv_rank + rot_dim padded to a
multiple of 16: every attention kernel of the engine serves it, and a cached token costs kv_rank + rot_dim elements
a plane.  The cache keeps that vector on both the key and the value plane of its page.

Parameters: ``hidden``, ``heads``, ``dim``, ``rot_dim``, ``v_head_dim``, ``q_rank``, ``kv_rank``, ``scale``, ``window``
(None: all keys), ``rotary_dims`` (0: no rotation), ``theta``, ``eps``, ``sink`` (learned, per head), ``gate``, ``names``.
"""
from __future__ import annotations

import torch

from ..cache.spec import CacheNeed
from ..config.registry import register_part
from ..weights.loader import TensorDecl
from .base import Mixer

_NAMES = {"dq": ".dq", "dq_norm": ".dq.norm", "uq": ".uq", "dkv": ".dkv", "dkv_norm": ".dkv.norm", "uk": ".uk", "uv": ".uv",
          "sink": ".sink", "gate": ".g", "out": ".o"}
MAX_HEAD = 512  # the widest cached vector the attention kernels take


class LatentAttention(Mixer):
    graph_safe = True  # reads the step's metadata on the device only

    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        p = params
        self.hidden, self.heads = int(p["hidden"]), int(p["heads"])
        self.dim, self.rot_dim, self.v_head_dim = int(p["dim"]), int(p["rot_dim"]), int(p["v_head_dim"])
        self.q_rank, self.kv_rank = int(p["q_rank"]), int(p["kv_rank"])
        self.scale, self.window, self.eps = float(p["scale"]), p.get("window"), float(p["eps"])
        self.rotary_dims, self.theta = int(p.get("rotary_dims") or 0), float(p.get("theta", 10000.0))
        if self.rotary_dims % 2 or self.rotary_dims > self.rot_dim:
            raise ValueError(f"rotary_dims {self.rotary_dims} must be even and at most rot_dim {self.rot_dim}")
        self.sink, self.gate = bool(p.get("sink", False)), bool(p.get("gate", False))
        self.names = {**_NAMES, **(p.get("names") or {})}
        self.latent = self.kv_rank + self.rot_dim                  # what a token caches
        self.padded = -(-self.latent // 16) * 16                   # the attention kernels' head size
        if self.padded > MAX_HEAD:
            raise ValueError(f"{prefix}: kv_rank + rot_dim = {self.latent} exceeds the attention kernels' {MAX_HEAD}")
        self.q_head = self.dim + self.rot_dim
        self.a_rows = self.q_rank + self.latent + (self.heads * self.v_head_dim if self.gate else 0)

    def activation_width(self):
        return max(self.a_rows, 2 * self.heads * self.padded + self.heads * self.kv_rank)

    def cache_need(self):
        return CacheNeed.kv(1, self.padded, self.window)

    def declare(self):
        pre, n, H = self.prefix, self.names, self.heads
        decls = [
            TensorDecl(pre + n["dq"], (self.q_rank, self.hidden)),
            TensorDecl(pre + n["dq_norm"], (self.q_rank,), init="ones"),
            TensorDecl(pre + n["uq"], (H * self.q_head, self.q_rank)),
            TensorDecl(pre + n["dkv"], (self.latent, self.hidden)),
            TensorDecl(pre + n["dkv_norm"], (self.kv_rank,), init="ones"),
            TensorDecl(pre + n["uk"], (H * self.dim, self.kv_rank)),
            TensorDecl(pre + n["uv"], (H * self.v_head_dim, self.kv_rank)),
            TensorDecl(pre + n["out"], (self.hidden, H * self.v_head_dim)),
        ]
        if self.sink:
            decls.append(TensorDecl(pre + n["sink"], (H,)))
        if self.gate:
            decls.append(TensorDecl(pre + n["gate"], (H * self.v_head_dim, self.hidden)))
        return decls

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        pre, n, H = self.prefix, self.names, self.heads
        t = lambda name: tensors[pre + n[name]]  # noqa: E731
        # one matrix for everything that reads the block's input: [dq; dkv; g]
        self.w_a = torch.cat([t("dq"), t("dkv")] + ([t("gate")] if self.gate else []), dim=0).contiguous()
        self.w_uq, self.w_out = t("uq").contiguous(), t("out").contiguous()
        # per head: W_uk as [kv_rank, dim] (it is applied to the query, transposed), W_uv as stored [v, kv_rank]
        self.w_uk_t = t("uk").view(H, self.dim, self.kv_rank).transpose(1, 2).contiguous()
        self.w_uv = t("uv").view(H, self.v_head_dim, self.kv_rank).contiguous()
        f32 = lambda name: t(name).to(torch.float32).contiguous()  # noqa: E731  (exact widening)
        self.dq_norm, self.dkv_norm = f32("dq_norm"), f32("dkv_norm")
        self.sink_values = f32("sink") if self.sink else None
        idx = torch.arange(0, self.rotary_dims, 2, dtype=torch.float64)
        # theta^(-2i / rotary_dims), taken in float64 and rounded once
        self.inv_freq = (torch.pow(torch.tensor(self.theta, dtype=torch.float64), -idx / max(self.rotary_dims, 1))
                         .to(torch.float32).to(rt.device).contiguous()) if self.rotary_dims else None

    def streamed_weights(self):
        return [self.w_a, self.w_uq, self.w_out]

    def forward(self, x, ctx, cache):
        ops, T, H, D = self.rt.ops, ctx.T, self.heads, self.padded
        a = ops.linear(x, self.w_a, meta=ctx.meta)
        cq = torch.empty((T, self.q_rank), dtype=x.dtype, device=x.device)
        ops.rms_rows(a[:, :self.q_rank], self.dq_norm, self.eps, cq, ctx.meta)
        q = ops.linear(cq, self.w_uq, meta=ctx.meta).view(T, H, self.q_head)
        q_abs = torch.empty((T, H, self.kv_rank), dtype=x.dtype, device=x.device)
        ops.head_linear(q[:, :, :self.dim], self.w_uk_t, q_abs, ctx.meta)
        q_full = torch.empty((T, H * D), dtype=x.dtype, device=x.device)
        ops.latent_rows(q[:, :, self.dim:], q_abs, a[:, self.q_rank:self.q_rank + self.latent], self.dkv_norm, self.eps, ctx,
                        cache.pages, cache.group, q_full, heads=H, kv_rank=self.kv_rank, rot_dim=self.rot_dim, padded=D,
                        page_size=cache.page_size, num_pages=cache.num_pages,
                        store=cache.writes and cache.pages is not None, inv_freq=self.inv_freq, rotary_dims=self.rotary_dims)
        out = torch.empty((T, H * D), dtype=x.dtype, device=x.device)
        ops.attention(q_full, H * D, cache.pages, ctx, cache.group, out, H, 1, D, cache.page_size, cache.num_pages,
                      int(self.window or 0), self.scale, sink=self.sink_values if self.sink else False)
        o = torch.empty((T, H, self.v_head_dim), dtype=x.dtype, device=x.device)
        gate = a[:, self.q_rank + self.latent:].view(T, H, self.v_head_dim) if self.gate else None
        ops.head_linear(out.view(T, H, D)[:, :, :self.kv_rank], self.w_uv, o, ctx.meta, gate=gate)
        return ops.linear(o.view(T, H * self.v_head_dim), self.w_out, meta=ctx.meta)


register_part("mixer", "latent_attention", LatentAttention)
