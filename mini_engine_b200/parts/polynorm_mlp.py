"""A dense feed-forward with the PolyNorm activation: ``down(act(up(x)))``,

``act(z) = a N(z) + b N(z^2) + c N(z^3) + e`` with powers element by element and N dividing a token's vector by its
root mean square (eps inside the root); the four numbers are a parameter of the layer.
"""
from __future__ import annotations

import torch

from .. import ops
from .base import FeedForward, ParamDecl
from .linear import Linear
from .registry import register_feed_forward


class PolyNormMLP(FeedForward):
    capturable = True

    def __init__(self, hidden_size: int, intermediate_size: int, eps: float, up: str = "up", down: str = "down", act: str = "act"):
        super().__init__()
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size
        self.eps = float(eps)
        self.act = act
        self.up_proj = Linear(hidden_size, [(up, intermediate_size)], name=up)
        self.down_proj = Linear(intermediate_size, [(down, hidden_size)], name=down)

    def sub_parts(self):
        return [("", self.up_proj), ("", self.down_proj)]

    def param_decls(self):
        return [ParamDecl(self.act, (4,), init="norm", role="vector")]

    def first_weight(self):
        return self.up_proj.weight

    def forward(self, x, ctx):
        z = self.up_proj.forward(x, ctx, "ffn_up", out_dtype=torch.float32)
        a = ctx.buffer("ffn_act", tuple(z.shape), ctx.act_dtype)
        ops.polynorm(z, self.p(self.act), self.eps, a)
        return self.down_proj.forward(a, ctx, "ffn_out")


register_feed_forward("polynorm_mlp", PolyNormMLP)
