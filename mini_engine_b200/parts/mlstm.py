"""The matrix memory of xLSTM (mLSTM) as a mixer with a state slot per request.

Per head: q = W_q h * dim^-1/2, k = W_k h (``dim`` values), v = W_v h (``vdim`` values), a log input gate
``i = cap tanh((W_i h + b_i) / cap)`` and a log forget gate ``f = logsigmoid(cap tanh((W_f h + b_f) / cap))``; then

    m_t = max(f + m_(t-1), i)                         (m starts at 0)
    S_t = exp(f + m_(t-1) - m_t) S_(t-1) + exp(i - m_t) k v^T,   n_t likewise with k alone
    o_t = S_t^T q / (max(|n_t . q|, exp(-m_t)) + 1e-6)

Each head's o is divided by its root mean square, the heads are concatenated, multiplied by a weight and by
sigmoid(W_g h), and projected by W_o.  S, n and m are float32 and live in the request's state slot; gates and
everything of the recurrence are float32 (the packed projection returns float32).
"""
from __future__ import annotations

import torch

from .. import ops
from .base import Mixer, ParamDecl, StateNeed
from .linear import Linear
from .registry import register_mixer


class MLSTM(Mixer):
    capturable = True

    def __init__(self, hidden_size: int, num_heads: int, dim: int, vdim: int, gate_cap: float, norm_eps: float):
        super().__init__()
        if not gate_cap > 0:
            raise ValueError(f"gate_cap must be positive, got {gate_cap}")
        self.hidden_size, self.num_heads, self.dim, self.vdim = hidden_size, num_heads, dim, vdim
        self.gate_cap = float(gate_cap)
        self.norm_eps = float(norm_eps)
        H = num_heads
        pieces = [("q", H * dim), ("k", H * dim), ("v", H * vdim), ("g", H * vdim), ("i", H), ("f", H)]
        self.in_proj = Linear(hidden_size, pieces, name="in_proj")
        self.offsets, off = {}, 0
        for name, rows in pieces:
            self.offsets[name] = off
            off += rows
        self.o_proj = Linear(H * vdim, [("o", hidden_size)], name="o")

    def sub_parts(self):
        return [("", self.in_proj), ("", self.o_proj)]

    def param_decls(self):
        H = self.num_heads
        return [ParamDecl("i.b", (H,), role="vector"), ParamDecl("f.b", (H,), init="norm", role="vector"),
                ParamDecl("norm", (H * self.vdim,), init="norm", role="vector")]

    def cache_needs(self):
        H, D, V = self.num_heads, self.dim, self.vdim
        return [StateNeed((H, D, V), "float32", "S"), StateNeed((H, D), "float32", "n"), StateNeed((H,), "float32", "m")]

    def first_weight(self):
        return self.in_proj.weight

    def forward(self, x, ctx, call):
        H, D, V = self.num_heads, self.dim, self.vdim
        proj = self.in_proj.forward(x, ctx, "mlstm_proj", out_dtype=torch.float32)
        T = proj.shape[0]
        o = ctx.buffer("mlstm_o", (T, H * V), torch.float32)
        slot = call.cache_slot
        ops.mlstm_scan(proj, self.offsets, self.p("i.b"), self.p("f.b"), self.gate_cap, ctx.state(slot, "S"), ctx.state(slot, "n"),
                       ctx.state(slot, "m"), ctx.attn_meta, ctx.state_slots, o, H, D, V, D ** -0.5)
        gated = ctx.buffer("mlstm_gated", (T, H * V), ctx.act_dtype)
        ops.mlstm_out(o, proj, self.offsets["g"], self.p("norm"), self.norm_eps, gated, H, V)
        return self.o_proj.forward(gated, ctx, "mixer_out")


register_mixer("mlstm", MLSTM)
