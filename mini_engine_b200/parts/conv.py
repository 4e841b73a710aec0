"""A short causal convolution over time on each channel, added to its input: ``h + conv(h)``.

``conv(h)_t = sum_j w[:, j] * h_(t - taps + 1 + j)`` for j = 0 .. taps-1 with zeros before a request's first token
(weight ``[channels, taps]``, no bias).  The last ``taps - 1`` inputs of a request are state: they live in the
request's state slot under the name the owner gives, so a request may be cut into portions anywhere.
"""
from __future__ import annotations

import torch

from .. import ops
from .base import ParamDecl, Part, StateNeed


class CausalShortConv(Part):
    capturable = True

    def __init__(self, channels: int, taps: int, param: str = "weight", state_name: str = "conv", residual: bool = True):
        super().__init__()
        if taps < 1:
            raise ValueError(f"a convolution needs at least one tap, got {taps}")
        self.channels = channels
        self.taps = taps
        self.param = param
        self.state_name = state_name
        self.residual = residual

    def param_decls(self):
        return [ParamDecl(self.param, (self.channels, self.taps), role="vector")]

    def cache_needs(self):
        if self.taps == 1:
            return []
        return [StateNeed((self.taps - 1, self.channels), "float32", self.state_name)]

    def forward(self, h: torch.Tensor, ctx, cache_slot: int, out_name: str = "conv_out") -> torch.Tensor:
        """``h`` [T, channels] float32 -> the working dtype."""
        out = ctx.buffer(out_name, tuple(h.shape), ctx.act_dtype)
        state = ctx.state(cache_slot, self.state_name) if self.taps > 1 else None
        ops.short_conv(h, self.p(self.param), state, ctx.token_req, ctx.attn_meta, ctx.state_slots, out, add_input=self.residual)
        return out
