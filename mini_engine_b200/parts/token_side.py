"""A layer's input from the token itself: a slice of a second embedding, gated by the residual stream.

e = table[token][first : first + dim]; g = gelu_tanh(W_gate x) * e; y = W_proj g.  What the block does with y (here: an
RMS norm with the plain weight ``norm`` and a scaled add) is the block's business; the part declares that weight.
The table belongs to the model and is shared by all layers, each with a slice of its own.
"""
from __future__ import annotations

import torch

from .. import ops
from .base import ParamDecl, Part
from .linear import Linear


class TokenSideInput(Part):
    capturable = True

    def __init__(self, hidden_size: int, dim: int, first: int, table, gate: str = "side.gate", proj: str = "side.proj",
                 norm: str = "side.norm"):
        super().__init__()
        self.hidden_size, self.dim, self.first = hidden_size, dim, first
        self.table = table                      # a part whose parameter is the table [vocab, columns]
        if first + dim > table.hidden_size:
            raise ValueError(f"slice [{first}, {first + dim}) is outside the table's {table.hidden_size} columns")
        self.gate = Linear(hidden_size, [(gate, dim)], name=gate)
        self.proj = Linear(dim, [(proj, hidden_size)], name=proj)
        self.norm = norm

    def sub_parts(self):
        return [("", self.gate), ("", self.proj)]

    def param_decls(self):
        return [ParamDecl(self.norm, (self.hidden_size,), init="norm", role="vector")]

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        """``x`` [T, hidden]: the residual stream in the working dtype -> y [T, hidden]."""
        z = self.gate.forward(x, ctx, "side_z", out_dtype=torch.float32)
        g = ctx.buffer("side_g", (x.shape[0], self.dim), ctx.act_dtype)
        ops.token_side_gate(z, ctx.token_ids, ctx.token_feedback, self.table.p(self.table.param), self.first, g)
        return self.proj.forward(g, ctx, "side_y")
