"""A plain, slow Logozen in float64 torch on the CPU: one function per mechanism, written from the design's equations.

It shares no code with the engine: weights are read straight from the safetensors file by their disk names, a
sequence is processed whole, every recurrence is a Python loop over tokens.  Notation: T tokens, W the model width,
H heads, streams s.
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
            w[name] = f.get_tensor(name).to(dtype)
    return cfg, w


# ---- small pieces ---------------------------------------------------------------------------------
def layer_norm(x, weight, eps):
    """(x - mean) / sqrt(var + eps) * weight over the last axis; var is the mean squared deviation; no bias."""
    mu = x.mean(-1, keepdim=True)
    d = x - mu
    return d / torch.sqrt((d * d).mean(-1, keepdim=True) + eps) * weight


def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))


def causal_conv_residual(h, taps_weight):
    """h + conv(h): conv(h)_t = sum_j w[:, j] * h_(t - taps + 1 + j), zeros before the sequence.  h [T, W], w [W, taps]."""
    T, W = h.shape
    taps = taps_weight.shape[1]
    out = h.clone()
    for t in range(T):
        for j in range(taps):
            src = t - taps + 1 + j
            if src >= 0:
                out[t] += taps_weight[:, j] * h[src]
    return out


def rotate_pairs(x, positions, base, dims):
    """Rotary positions, interleaved pairs (2i, 2i+1), on the first ``dims`` elements of the last axis.
    x [T, ..., D]; positions [T]."""
    out = x.clone()
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        a = positions.to(x.dtype) * f
        shape = [-1] + [1] * (x.dim() - 2)
        c, s = torch.cos(a).view(shape), torch.sin(a).view(shape)
        u, v = x[..., 2 * i], x[..., 2 * i + 1]
        out[..., 2 * i] = u * c - v * s
        out[..., 2 * i + 1] = v * c + u * s
    return out


# ---- mixers ------------------------------------------------------------------------------------------
def latent_attention(h, w, pre, m, eps):
    """Attention through a low-rank latent with one shared rotated key part, a sink in the softmax and a gate per head."""
    T = h.shape[0]
    H, D, R, V, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    q = (h @ w[pre + "q"].T).view(T, H, D + R)
    q_plain, q_rot = q[..., :D], rotate_pairs(q[..., D:], pos, m["rot"]["base"], m["rot"]["dims"])
    dkv = h @ w[pre + "dkv"].T
    c = unit_rms(dkv[:, :C], eps) * w[pre + "dkv.norm"]
    k_rot = rotate_pairs(dkv[:, C:], pos, m["rot"]["base"], m["rot"]["dims"])          # [T, R], shared by the heads
    k_plain = (c @ w[pre + "uk"].T).view(T, H, D)
    v = (c @ w[pre + "uv"].T).view(T, H, V)
    gate = torch.sigmoid(h @ w[pre + "g"].T)                                             # [T, H]
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for hd in range(H):
        s = (q_plain[:, hd] @ k_plain[:, hd].T + q_rot[:, hd] @ k_rot.T) * m["scale"]   # [T, T]
        s = s.masked_fill(torch.arange(T)[None, :] > torch.arange(T)[:, None], float("-inf"))
        sink = w[pre + "sink"][hd]
        mx = torch.maximum(s.max(-1, keepdim=True).values, sink)
        e = torch.exp(s - mx)
        p = e / (e.sum(-1, keepdim=True) + torch.exp(sink - mx))
        out[:, hd] = (p @ v[:, hd]) * gate[:, hd:hd + 1]
    return out.reshape(T, H * V) @ w[pre + "o"].T


def mlstm(h, w, pre, m, eps):
    """Matrix-memory recurrence with capped gates, a running maximum that starts at 0, and a per-head unit-RMS output."""
    T = h.shape[0]
    H, D, V, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    q = (h @ w[pre + "q"].T).view(T, H, D) * D ** -0.5
    k = (h @ w[pre + "k"].T).view(T, H, D)
    v = (h @ w[pre + "v"].T).view(T, H, V)
    gi = cap * torch.tanh((h @ w[pre + "i"].T + w[pre + "i.b"]) / cap)
    gf = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ w[pre + "f"].T + w[pre + "f.b"]) / cap))
    S = torch.zeros(H, D, V, dtype=h.dtype)
    n = torch.zeros(H, D, dtype=h.dtype)
    mx = torch.zeros(H, dtype=h.dtype)
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for t in range(T):
        m_new = torch.maximum(gf[t] + mx, gi[t])
        a = torch.exp(gf[t] + mx - m_new)
        b = torch.exp(gi[t] - m_new)
        S = a[:, None, None] * S + b[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = a[:, None] * n + b[:, None] * k[t]
        mx = m_new
        num = torch.einsum("hdv,hd->hv", S, q[t])
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-mx)) + 1e-6
        out[t] = num / den[:, None]
    out = unit_rms(out, eps).reshape(T, H * V) * w[pre + "norm"]
    out = out * torch.sigmoid(h @ w[pre + "g"].T)
    return out @ w[pre + "o"].T


MIXERS = {"latent_attention": latent_attention, "mlstm": mlstm}


# ---- feed-forward -------------------------------------------------------------------------------------
def polynorm_feed_forward(h, w, pre, eps):
    z = h @ w[pre + "up"].T
    a, b, c, e = w[pre + "act"]
    act = a * unit_rms(z, eps) + b * unit_rms(z ** 2, eps) + c * unit_rms(z ** 3, eps) + e
    return act @ w[pre + "down"].T


# ---- the model -----------------------------------------------------------------------------------------
def hyper_sublayer(streams, hc_in, hc_mix, hc_out, sublayer):
    """streams [s, T, W].  u = sum_s in[s] x_s; y = sublayer(u); x_t <- sum_s mix[s, t] x_s + out[t] y."""
    u = torch.einsum("s,stw->tw", hc_in, streams)
    y = sublayer(u)
    return torch.einsum("sr,stw->rtw", hc_mix, streams) + hc_out[:, None, None] * y[None]


def forward(cfg, w, ids, return_layers=False):
    """Logits [T, vocab] of one whole sequence (and the sum of the streams after every layer, if asked)."""
    dtype = w["embed"].dtype
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.tensor(ids)] * cfg["embedding"]["scale"]
    streams = x[None].repeat(cfg["streams"], 1, 1)
    after = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        mixer = MIXERS[layer["type"]]

        def mix(u, p=p, layer=layer, mixer=mixer):
            h = causal_conv_residual(layer_norm(u, w[p + "norm1"], eps), w[p + "canon1"])
            return mixer(h, w, p + "mix.", layer["mixer"], eps)
        streams = hyper_sublayer(streams, w[p + "hc1.in"], w[p + "hc1.mix"], w[p + "hc1.out"], mix)
        if layer.get("mlp") is not None:
            if layer["mlp"]["kind"] != "dense":
                raise ValueError(f"unknown feed-forward kind {layer['mlp']['kind']!r}")

            def ff(u, p=p):
                h = causal_conv_residual(layer_norm(u, w[p + "norm2"], eps), w[p + "canon2"])
                return polynorm_feed_forward(h, w, p + "mlp.", eps)
            streams = hyper_sublayer(streams, w[p + "hc2.in"], w[p + "hc2.mix"], w[p + "hc2.out"], ff)
        after.append(streams.sum(0))
    x = layer_norm(streams.sum(0), w["final.norm"], eps)
    logits = x @ w["head"].T
    return (logits, torch.stack(after)) if return_layers else logits


def forward_logits(cfg, w, ids):
    return forward(cfg, w, ids).to(torch.float32)
