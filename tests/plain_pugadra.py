"""A plain, slow Pugadra in float64 torch on the CPU: one function per mechanism, written from the design's equations.

It shares no code with the engine: weights are a dict from disk names to tensors, a sequence is processed whole, the
attention is a loop over queries.  Notation: T tokens, W the model width, H query heads, G key/value heads.
"""
from __future__ import annotations

import json
import math
import os

import torch
from safetensors import safe_open


def load_folder(folder: str, dtype=torch.float64):
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    w = {}
    with safe_open(os.path.join(folder, "model.safetensors"), "pt", device="cpu") as f:
        for name in f.keys():
            t = f.get_tensor(name)
            w[name] = t.to(dtype) if t.is_floating_point() else t
    return cfg, w


# ---- small pieces ---------------------------------------------------------------------------------
def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_around_zero(x, weight, eps):
    """The model's norm: the weight is stored as its distance from one."""
    return unit_rms(x, eps) * (1 + weight)


def norm_plain_weight(x, weight, eps):
    return unit_rms(x, eps) * weight


def gelu_tanh(z):
    return 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))


def causal_conv(u, taps_weight):
    """y_t = sum_j w[:, j] * u_(t - taps + 1 + j), zeros before the sequence.  u [T, C], w [C, taps]."""
    T, C = u.shape
    taps = taps_weight.shape[1]
    out = torch.zeros_like(u)
    for t in range(T):
        for j in range(taps):
            src = t - taps + 1 + j
            if src >= 0:
                out[t] += taps_weight[:, j] * u[src]
    return out


def rotate_pairs(x, positions, base, dims):
    """Rotary positions on neighbouring pairs (2i, 2i+1) of the first ``dims`` elements of the last axis.
    x [T, heads, D]; positions [T]."""
    out = x.clone()
    for i in range(dims // 2):
        a = positions.to(x.dtype) * base ** (-2.0 * i / dims)
        c, s = torch.cos(a)[:, None], torch.sin(a)[:, None]
        u, v = x[..., 2 * i], x[..., 2 * i + 1]
        out[..., 2 * i] = u * c - v * s
        out[..., 2 * i + 1] = v * c + u * s
    return out


def windowed_sink_attention(q, k, v, scale, window):
    """q [T, H, D], k [T, G, D], v [T, G, Dv] -> [T, H, Dv].  Query i sees keys j with 0 <= i - j < window (all j <= i
    when window is None); the weights are exp(s_j) / (1 + sum exp(s_j)): a sink of score 0 that has no value."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for i in range(T):
        lo = 0 if window is None else max(0, i - window + 1)
        for h in range(H):
            g = h // (H // G)
            s = (k[lo:i + 1, g] @ q[i, h]) * scale
            m = max(float(s.max()), 0.0)
            e = torch.exp(s - m)
            out[i, h] = (e[:, None] * v[lo:i + 1, g]).sum(0) / (math.exp(-m) + e.sum())
    return out


def clamped_glu(h, w, pre, limit):
    """g = min(W_gate h, limit), u = clamp(W_up h, -limit, limit), y = g sigmoid(1.702 g) (u + 1), out = W_down y
    (``limit`` None: nothing is clamped)."""
    g, u = h @ w[pre + "gate"].T, h @ w[pre + "up"].T
    if limit is not None:
        g, u = g.clamp(max=limit), u.clamp(-limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1)) @ w[pre + "down"].T


# ---- sub-layers ------------------------------------------------------------------------------------
def attention_keys_values(h, w, pre, m, positions):
    """The keys (after convolution and rotation) and values (after convolution) that a layer computes and caches."""
    T = h.shape[0]
    G, D, Dv = m["kv_heads"], m["dim"], m["vdim"]
    k = h @ w[pre + "k"].T + w[pre + "k.b"]
    v = h @ w[pre + "v"].T + w[pre + "v.b"]
    if m.get("conv"):
        k, v = causal_conv(k, w[pre + "k.conv"]), causal_conv(v, w[pre + "v.conv"])
    k = k.view(T, G, D)
    if m.get("rot"):
        k = rotate_pairs(k, positions, m["rot"]["base"], m["rot"]["dims"])
    return k, v.view(T, G, Dv)


def attention(h, w, pre, m, kv):
    """``kv``: the keys and values to use (this layer's own, or those of the layer it takes them from)."""
    T = h.shape[0]
    H, D, Dv = m["heads"], m["dim"], m["vdim"]
    positions = torch.arange(T)
    q = h @ w[pre + "q"].T + w[pre + "q.b"]
    if m.get("conv"):
        q = causal_conv(q, w[pre + "q.conv"])
    q = q.view(T, H, D)
    if m.get("rot"):
        q = rotate_pairs(q, positions, m["rot"]["base"], m["rot"]["dims"])
    k, v = kv
    window = m["mask"]["size"] if m.get("mask") else None
    o = windowed_sink_attention(q, k, v, m["scale"], window).reshape(T, H * Dv)
    o = o * torch.sigmoid(h @ w[pre + "g"].T)
    return o @ w[pre + "o"].T


def routed_experts(h, w, pre, mlp):
    """Top-k routing: softmax over the chosen logits only; plus the shared expert, if there is one."""
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    z = h @ w[pre + "router"].T + w[pre + "router.b"]
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        chosen = torch.topk(z[t], top).indices
        p = torch.softmax(z[t, chosen], 0)
        for e, pe in zip(chosen.tolist(), p):
            out[t] += pe * clamped_glu(h[t:t + 1], w, f"{pre}e{e}.", mlp["expert"].get("limit"))[0]
    if mlp.get("shared"):
        out = out + clamped_glu(h, w, pre + "shared.", mlp["shared"].get("limit"))
    return out


def feed_forward(h, w, pre, mlp):
    if mlp["kind"] == "dense":
        return clamped_glu(h, w, pre, mlp.get("limit"))
    return routed_experts(h, w, pre, mlp)


def token_side_input(x, tokens, w, pre, layer, dim, eps):
    """What a layer adds from the token itself: a slice of a second embedding, gated by the stream."""
    e = w["side.embed"][tokens][:, layer * dim:(layer + 1) * dim]
    y = (gelu_tanh(x @ w[pre + "side.gate"].T) * e) @ w[pre + "side.proj"].T
    return norm_plain_weight(y, w[pre + "side.norm"], eps)


# ---- the model ---------------------------------------------------------------------------------------
def forward(cfg, w, tokens, return_layers=False):
    """Logits [T, vocab] for one sequence (and, if asked, the residual stream after every layer)."""
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    eps, mult = cfg["norm"]["eps"], cfg["residual_mult"]
    side_dim = cfg["token_side"]["dim"] if cfg.get("token_side") else 0
    x = w["embed"][tokens]
    positions = torch.arange(len(tokens))
    cached, after = {}, []
    for i, layer in enumerate(cfg["layers"]):
        pre, m = f"l{i}.", layer["mixer"]
        h = norm_around_zero(x, w[pre + "norm1"], eps)
        if m.get("kv_from") is None:
            cached[i] = attention_keys_values(h, w, pre + "mix.", m, positions)
        y = attention(h, w, pre + "mix.", m, cached[m["kv_from"] if m.get("kv_from") is not None else i])
        x = x + mult * norm_around_zero(y, w[pre + "norm1b"], eps)
        if layer.get("mlp") is not None:
            y = feed_forward(norm_around_zero(x, w[pre + "norm2"], eps), w, pre + "mlp.", layer["mlp"])
            x = x + mult * norm_around_zero(y, w[pre + "norm2b"], eps)
        if side_dim:
            x = x + mult * token_side_input(x, tokens, w, pre, i, side_dim, eps)
        after.append(x)
    logits = norm_around_zero(x, w["final.norm"], eps) @ w["embed"].T
    return (logits, torch.stack(after)) if return_layers else logits
