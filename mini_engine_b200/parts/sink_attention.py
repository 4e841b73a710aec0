"""Grouped-query attention with a window, a sink in the softmax, convolved projections and an output gate.

q = W_q h + b_q, k = W_k h + b_k, v = W_v h + b_v (biases optional); a short causal convolution over time on every
channel of q, k and v directly behind the projection (``conv_taps`` taps, no bias; the last taps - 1 projected values of
a request are its state); rotary positions on neighbouring pairs of the first ``rotary_dim`` elements of each q and k
head; score = q . k * scale; a query at position p sees keys p - window < j <= p (all j <= p without a window); the
weights are exp(s_j) / (sink + sum exp(s_j)) with sink = 1 when ``sink`` is set (a key of score 0 that has no value);
the concatenated heads are multiplied by sigmoid(W_g h) when ``gate`` is set; then the output projection.  Keys have
``dim`` elements and values ``vdim``; the cache is the engine's usual one (pages of keys and of values) with rows of
max(dim, vdim) elements, so that equal sizes of 64 or 128 run the engine's tensor-core attention kernels.

``own_kv`` False: the mixer has no key and value projections; it reads the cache rows of another call (``call.kv_slot``)
with its own queries, window and everything else.  ``cache_window``: what the cache must keep for all mixers that read
this one's rows (the widest of their windows, None when one of them sees every key).

Scores, softmax, angles and the rotation are float32; the packed projection returns float32, so the convolution, its
state, the rotation and the gate see unrounded sums.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from .base import DiskSource, KVCacheNeed, Mixer, ParamDecl, StateNeed
from .linear import Linear
from .registry import PartSpec, build_part, register_mixer


class SinkAttention(Mixer):
    capturable = True

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, dim: int, vdim: int, scale: float,
                 position_encoding: Optional[PartSpec | object] = None, window: Optional[int] = None,
                 cache_window: Optional[int] = None, conv_taps: Optional[int] = None, bias: bool = True, gate: bool = True, sink: bool = True,
                 own_kv: bool = True):
        super().__init__()
        if num_heads < 1 or num_kv_heads < 1 or num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads are no multiple of {num_kv_heads} kv heads")
        self.hidden_size, self.num_heads, self.num_kv_heads = hidden_size, num_heads, num_kv_heads
        self.dim, self.vdim = dim, vdim
        self.scale = float(scale)
        self.window, self.cache_window = window, cache_window
        self.taps = int(conv_taps or 0)         # 0: no convolution; 1: a weight per channel and no state
        self.has_bias, self.has_gate, self.has_sink, self.own_kv = bias, gate, sink, own_kv
        if isinstance(position_encoding, PartSpec):
            position_encoding = build_part("position_encoding", position_encoding)
        self.rope = position_encoding
        if self.rope is not None and (self.rope.layout != "interleaved" or self.rope.rotary_dim > dim or dim % 2):
            raise ValueError("SinkAttention rotates neighbouring pairs of at most dim elements of an even head size "
                             f"(got layout {self.rope.layout!r}, {self.rope.rotary_dim} of {dim})")
        H, G = num_heads, num_kv_heads
        self.pieces = [("q", H * dim)] + ([("k", G * dim), ("v", G * vdim)] if own_kv else [])
        self.channels = sum(n for _, n in self.pieces)        # what passes through bias, convolution and rotation
        self.in_proj = Linear(hidden_size, self.pieces + ([("g", H * vdim)] if gate else []), name="in_proj")
        self.o_proj = Linear(H * vdim, [("o", hidden_size)], name="o")
        self._no_freq = None

    def sub_parts(self):
        parts = [("", self.in_proj), ("", self.o_proj)]
        if self.rope is not None:
            parts.append(("rot.", self.rope))
        return parts

    def _packed(self, name: str, suffix: str, shape_tail: tuple[int, ...]) -> ParamDecl:
        sources, start = [], 0
        for piece, n in self.pieces:
            sources.append(DiskSource(piece + suffix, start, n))
            start += n
        return ParamDecl(name, (self.channels, *shape_tail), sources=sources, role="vector")

    def param_decls(self):
        decls = []
        if self.has_bias:
            decls.append(self._packed("in_bias", ".b", ()))
        if self.taps >= 1:
            decls.append(self._packed("in_conv", ".conv", (self.taps,)))
        return decls

    def cache_needs(self):
        needs = [KVCacheNeed(self.num_kv_heads, max(self.dim, self.vdim), self.cache_window)] if self.own_kv else []
        if self.taps > 1:
            needs.append(StateNeed((self.taps - 1, self.channels), "float32", "conv"))
        return needs

    def first_weight(self):
        return self.in_proj.weight

    def finalize(self, dtype, device):
        self._no_freq = torch.zeros(0, dtype=torch.float64, device=device)

    def forward(self, x, ctx, call):
        H, G, D, V = self.num_heads, self.num_kv_heads, self.dim, self.vdim
        proj = self.in_proj.forward(x, ctx, "attn_proj", out_dtype=torch.float32)
        T = proj.shape[0]
        kv = ctx.kv_cache(call.cache_slot if self.own_kv else call.kv_slot)
        q = ctx.buffer("attn_q", (T, H * D), ctx.act_dtype)
        inv_freq = self.rope.inv_freq if self.rope is not None else self._no_freq
        angles = None
        if self.rope is not None and T >= ops.ROPE_TABLE_MIN_TOKENS:
            # One table for all layers that share the rotation, made anew in every pass over the layers (a pass that is being
            # recorded into a graph must launch it too, or the replay would rotate by the positions of the recording).
            cache = getattr(ctx, "_rope_tables", None)
            if cache is None or cache[0] != ctx.forward_serial:
                cache = ctx._rope_tables = (ctx.forward_serial, {})
            tables = cache[1]
            angles = tables.get(id(self.rope))
            if angles is None:
                angles = tables[id(self.rope)] = ctx.buffer(f"rope_table_{self.rope.rotary_dim}_{self.rope.theta!r}",
                                                            (T, inv_freq.numel(), 2), torch.float32)
                ops.rope_table(ctx.positions, inv_freq, angles)
        ops.conv_rope_kv(proj, self.p("in_bias") if self.has_bias else None, self.p("in_conv") if self.taps >= 1 else None,
                         ctx.state(call.cache_slot, "conv") if self.taps > 1 else None, inv_freq, inv_freq.numel() * 2, ctx,
                         kv.slot_mapping if self.own_kv and call.writes_cache else None, q, kv.pool, kv.page_size, H, G, D, V,
                         self.own_kv and call.writes_cache, angles=angles)
        out = ctx.buffer("attn_out", (T, H * V), ctx.act_dtype)
        gate = proj[:, self.channels:] if self.has_gate else None
        ops.sink_attention(q, gate, out, kv.pool, kv.page_size, kv.block_tables, ctx.attn_meta, H, G, D, V, self.scale,
                           self.window, self.has_sink)
        return self.o_proj.forward(out, ctx, "mixer_out")


register_mixer("sink_attention", SinkAttention)
