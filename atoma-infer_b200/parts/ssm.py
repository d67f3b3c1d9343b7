"""Mamba-2 mixer: a state-space recurrence per head, fed through one input projection and a short causal convolution.

With inner = heads * head_dim, N = state and G = groups, the input projection's rows are [z: inner | x: inner |
B: G*N | C: G*N | dt: heads].  x, B and C pass a causal convolution over time on each channel (weights [channels,
taps], a bias, zeros before the request's start) and SiLU.  dt <- softplus(dt + dt_bias).  Head h (of group
h // (heads / G)) keeps a matrix S of N x head_dim: S_t = exp(-exp(A_log_h) dt_t) S_(t-1) + dt_t B_t x_t^T,
y_t = S_t^T C_t + D_h x_t.  The heads' y, times SiLU(z), are divided in ``norm_groups`` equal parts by each part's
root mean square, multiplied by a weight, and projected out.

State per request (float32, fixed size, ``cache.state[slot]``): the convolution's last taps - 1 input rows as a
ring (the row of position p at place p mod (taps - 1), so a row's place does not depend on how the prompt was cut),
then the heads' matrices.  Softplus, decays, the recurrence, the gate and the norm are float32 in every mode; the
projections, the convolution and its activation run in the compute dtype.

Parameters: ``hidden``, ``heads``, ``head_dim``, ``state``, ``groups``, ``taps``, ``norm_groups``, ``eps``, ``names``
(suffixes of the tensors: in, conv, conv_bias, dt_bias, a_log, d, norm, out).
"""
from __future__ import annotations

import torch

from ..config.registry import register_part
from ..weights.loader import TensorDecl
from .base import Mixer

_NAMES = {"in": ".in", "conv": ".conv", "conv_bias": ".conv.b", "dt_bias": ".dt_bias", "a_log": ".A_log", "d": ".D",
          "norm": ".norm", "out": ".o"}


class Mamba2Mixer(Mixer):
    graph_safe = True  # reads the step's metadata on the device only

    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        p = params
        self.hidden, self.heads, self.head_dim = int(p["hidden"]), int(p["heads"]), int(p["head_dim"])
        self.nstate, self.groups, self.taps = int(p["state"]), int(p.get("groups", 1)), int(p["taps"])
        self.norm_groups, self.eps = int(p.get("norm_groups", 1)), float(p["eps"])
        if self.heads % self.groups:
            raise ValueError("heads must be a multiple of groups")
        self.inner = self.heads * self.head_dim
        if self.inner % self.norm_groups:
            raise ValueError("norm_groups must divide heads * head_dim")
        self.channels = self.inner + 2 * self.groups * self.nstate   # what the convolution sees: x, B, C
        self.proj = 2 * self.inner + 2 * self.groups * self.nstate + self.heads
        self.names = {**_NAMES, **(p.get("names") or {})}
        # the state's two shares, each starting on 16 bytes
        self.ring_bytes = -(-(self.taps - 1) * self.channels * 4 // 16) * 16
        self.matrix_bytes = self.heads * self.nstate * self.head_dim * 4

    def activation_width(self):
        return self.proj + 2 * self.channels

    def state_bytes(self):
        return self.ring_bytes + self.matrix_bytes

    def declare(self):
        pre, n = self.prefix, self.names
        return [
            TensorDecl(pre + n["in"], (self.proj, self.hidden)),
            TensorDecl(pre + n["conv"], (self.channels, self.taps)),
            TensorDecl(pre + n["conv_bias"], (self.channels,)),
            TensorDecl(pre + n["dt_bias"], (self.heads,)),
            TensorDecl(pre + n["a_log"], (self.heads,)),
            TensorDecl(pre + n["d"], (self.heads,), init="ones"),
            TensorDecl(pre + n["norm"], (self.inner,), init="ones"),
            TensorDecl(pre + n["out"], (self.hidden, self.inner)),
        ]

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        pre, n = self.prefix, self.names
        f32 = lambda name: tensors[pre + n[name]].to(torch.float32).contiguous()  # noqa: E731  (exact widening)
        self.w_in, self.w_out = tensors[pre + n["in"]].contiguous(), tensors[pre + n["out"]].contiguous()
        # [taps, channels]: neighbouring threads of the kernels read neighbouring weights
        self.conv_w = tensors[pre + n["conv"]].to(torch.float32).t().contiguous()
        self.conv_b, self.dt_bias, self.a_log, self.d_skip, self.norm_w = (f32(k) for k in ("conv_bias", "dt_bias", "a_log", "d", "norm"))

    def streamed_weights(self):
        return [self.w_in, self.w_out]

    def ring(self, state):
        """The convolution's share of the state: float32 [slots, taps - 1, channels] (None with one tap)."""
        if state is None or self.taps == 1:
            return None
        return state[:, :(self.taps - 1) * self.channels * 4].view(torch.float32).view(state.shape[0], self.taps - 1, self.channels)

    def matrices(self, state):
        """The recurrence's share of the state: float32 [slots, heads, N, head_dim]."""
        return state[:, self.ring_bytes:self.ring_bytes + self.matrix_bytes].view(torch.float32).view(
            state.shape[0], self.heads, self.nstate, self.head_dim)

    def forward(self, x, ctx, cache):
        ops, T, inner = self.rt.ops, ctx.T, self.inner
        proj = ops.linear(x, self.w_in, meta=ctx.meta)
        z, u, dt = proj[:, :inner], proj[:, inner:inner + self.channels], proj[:, inner + self.channels:]
        ring = self.ring(cache.state)
        xbc = torch.empty((T, self.channels), dtype=x.dtype, device=x.device)
        if not ops.causal_conv_act(u, self.conv_w, self.conv_b, ring, ctx, xbc, act="silu"):
            ops.causal_conv_save(u, ring, ctx, self.taps)  # after the convolution has read the ring
        y = torch.empty((T, inner), dtype=torch.float32, device=x.device)
        ops.ssm_scan(xbc, dt, self.dt_bias, self.a_log, self.d_skip, self.matrices(cache.state), ctx, y,
                     heads=self.heads, head_dim=self.head_dim, nstate=self.nstate, groups=self.groups)
        g = torch.empty((T, inner), dtype=x.dtype, device=x.device)
        ops.gated_group_norm(y, z, self.norm_w, self.norm_groups, self.eps, g, ctx.meta)
        return ops.linear(g, self.w_out, meta=ctx.meta)


register_part("mixer", "mamba2", Mamba2Mixer)
