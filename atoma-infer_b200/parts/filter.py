"""Short causal convolution over time in front of a sublayer: the sublayer reads h + conv(h) instead of h, with
conv(h)_t = sum_j w[:, j] * h_(t - taps + 1 + j) on each channel and zeros before the request's start.

The last ``taps - 1`` rows a request fed in are its state: float32, one ring per state slot in which the row of
position p lies at place p mod (taps - 1), so that a step of any length finds the rows before its portion and a
row's place does not depend on how the prompt was cut.

Parameters: ``channels``, ``taps``, ``add_input`` (True: h + conv(h); False: conv(h) alone).  Checkpoint tensor:
``<prefix>`` of shape [channels, taps], no bias.
"""
from __future__ import annotations

import torch

from ..config.registry import register_part
from ..weights.loader import TensorDecl
from .base import SequenceFilter


class ShortConv(SequenceFilter):
    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        self.channels, self.taps = int(params["channels"]), int(params["taps"])
        self.add_input = bool(params.get("add_input", True))
        if self.taps < 1:
            raise ValueError("a short convolution needs at least one tap")

    def declare(self):
        return [TensorDecl(self.prefix, (self.channels, self.taps))]

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        # widened exactly; kept as [taps, channels] so that neighbouring threads of the kernels read neighbouring weights
        self.weight = tensors[self.prefix].to(torch.float32).t().contiguous()

    def state_bytes(self):
        return (self.taps - 1) * self.channels * 4

    def ring(self, state):
        """The part's share of the state as float32 [slots, taps - 1, channels] (None with one tap)."""
        if state is None or self.taps == 1:
            return None
        return state.view(torch.float32).view(state.shape[0], self.taps - 1, self.channels)

    def fused(self):
        return {"kind": "short_conv", "weight": self.weight, "taps": self.taps, "add_input": self.add_input}

    def forward(self, resid, ctx, state):
        out = torch.empty((ctx.T, self.channels), dtype=self.rt.dtype, device=resid.device)
        self.rt.ops.short_conv(resid, self.weight, self.ring(state), ctx, out, add_input=self.add_input)
        return out

    def save(self, resid, ctx, state):
        self.rt.ops.short_conv_save(resid, self.ring(state), ctx, self.taps)


register_part("filter", "short_conv", ShortConv)
