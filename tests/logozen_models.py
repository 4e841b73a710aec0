"""Small Logozen models for the tests: configurations that differ in every size and constant, and random weights.

The writer here knows the tensor names and shapes of the design by itself (it does not ask the engine), draws
matrices as N(0, gain / sqrt(inputs)) so that every layer changes the residual streams noticeably, and lets a test
overwrite any tensor before the folder is written.
"""
from __future__ import annotations

import functools
import json
import os
import tempfile

import torch
from safetensors.torch import save_file


def latent(heads, dim, rot_dim, vdim, kv_rank, rot_dims=None, base=10000.0, scale=None, ff=None):
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
                      "rot": {"base": base, "dims": rot_dim if rot_dims is None else rot_dims},
                      "scale": (dim + rot_dim) ** -0.5 if scale is None else scale},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def mlstm(heads, dim, vdim, gate_cap=15.0, ff=None):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": gate_cap},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def config(vocab, width, streams, taps, layers, eps=1e-5, embed_scale=1.0):
    return {"architecture": "Logozen", "vocab": vocab, "width": width, "streams": streams, "canon": {"taps": taps},
            "embedding": {"scale": embed_scale}, "norm": {"eps": eps}, "layers": layers}


# P: three streams, four taps, odd sizes, only part of the rotated dimensions rotated, a layer without feed-forward,
#    a value size that is no multiple of 32
P = config(97, 48, 3, 4, [
    latent(3, 16, 8, 24, 40, rot_dims=4, base=5000.0, ff=72),
    mlstm(2, 24, 40, gate_cap=8.0, ff=None),
    latent(3, 16, 8, 24, 40, rot_dims=4, base=5000.0, ff=None),
    mlstm(2, 24, 40, gate_cap=8.0, ff=88),
], eps=1e-6, embed_scale=7.0)
# Q: ONE stream and ONE tap (no state for the convolution), attention first, 20 heads (two blocks of heads in decoding),
#    two different rotations, scale not tied to the sizes
Q = config(160, 64, 1, 1, [
    latent(20, 8, 4, 8, 16, base=100.0, scale=0.3, ff=96),
    mlstm(4, 8, 16, gate_cap=20.0, ff=96),
    latent(2, 32, 16, 32, 24, base=1e6, ff=None),
], eps=3e-5, embed_scale=1.0)
# R: the recurrence alone (a model without any paged cache), two taps, five streams
R = config(64, 40, 5, 2, [mlstm(3, 16, 32, gate_cap=10.0, ff=56), mlstm(1, 40, 72, gate_cap=10.0, ff=None)],
           eps=1e-5, embed_scale=3.0)
# S: attention alone, eight streams, three taps, a latent wider than 128 (the kernel's second form)
S = config(80, 56, 8, 3, [latent(4, 24, 8, 16, 136, ff=64), latent(4, 24, 8, 16, 136, ff=None)], eps=1e-5, embed_scale=2.5)

# U: no size a multiple of 8 (width, feed-forward, heads' sizes, latent), eleven streams, seven taps, six rotated of ten dims
U = config(75, 52, 11, 7, [mlstm(5, 12, 20, gate_cap=30.0, ff=70), latent(5, 10, 10, 12, 20, rot_dims=6, base=300.0, ff=70),
                            latent(7, 6, 2, 9, 13, base=50.0, ff=None)], eps=2e-5, embed_scale=5.0)

ALL = {"P": (P, 1, 16), "Q": (Q, 2, 8), "R": (R, 3, 16), "S": (S, 4, 32), "U": (U, 5, 16)}        # config, seed, page size


def tensors(cfg: dict, seed: int, gain: float = 1.2) -> dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    W, S, taps = cfg["width"], cfg["streams"], cfg["canon"]["taps"]

    def mat(rows, cols, k=gain):
        return torch.randn(rows, cols, generator=g) * (k / cols ** 0.5)

    def around(n, mean, std):
        return mean + std * torch.randn(n, generator=g)
    t = {"embed": torch.randn(cfg["vocab"], W, generator=g) * 0.08, "head": mat(cfg["vocab"], W, 1.0),
         "final.norm": around(W, 0.9, 0.3)}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        H = m["heads"]
        subs = ("1", "2") if layer["mlp"] is not None else ("1",)
        for q in subs:
            t[p + "norm" + q] = around(W, 1.0, 0.2)
            t[p + "canon" + q] = torch.randn(W, taps, generator=g) * 0.35
            t[p + f"hc{q}.in"] = around(S, 1.2 / S, 0.3 / S)
            t[p + f"hc{q}.out"] = around(S, 0.9, 0.25)
            t[p + f"hc{q}.mix"] = torch.eye(S) + 0.15 * torch.randn(S, S, generator=g)
        if layer["type"] == "latent_attention":
            D, R, V, C = m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            t[p + "mix.q"] = mat(H * (D + R), W, 1.4)
            t[p + "mix.dkv"] = mat(C + R, W, 1.4)
            t[p + "mix.dkv.norm"] = around(C, 1.0, 0.15)
            t[p + "mix.uk"] = mat(H * D, C, 1.3)
            t[p + "mix.uv"] = mat(H * V, C, 1.5)
            t[p + "mix.sink"] = around(H, 2.0, 1.0)
            t[p + "mix.g"] = mat(H, W, 1.4)
            t[p + "mix.o"] = mat(W, H * V, 1.3)
        else:
            D, V = m["dim"], m["vdim"]
            t[p + "mix.q"], t[p + "mix.k"] = mat(H * D, W), mat(H * D, W)
            t[p + "mix.v"], t[p + "mix.g"] = mat(H * V, W), mat(H * V, W, 1.5)
            t[p + "mix.o"] = mat(W, H * V, 1.0)
            t[p + "mix.norm"] = around(H * V, 1.0, 0.2)
            t[p + "mix.i"], t[p + "mix.f"] = mat(H, W, 0.9), mat(H, W, 0.9)
            t[p + "mix.i.b"] = around(H, 0.0, 1.0)
            t[p + "mix.f.b"] = around(H, 3.0, 1.5)
        if layer["mlp"] is not None:
            F = layer["mlp"]["ff"]
            t[p + "mlp.up"], t[p + "mlp.down"] = mat(F, W, 1.3), mat(W, F, 0.9)
            t[p + "mlp.act"] = around(4, 0.6, 0.25)
    return {k: v.to(torch.bfloat16).contiguous() for k, v in t.items()}


def write_folder(cfg: dict, weights: dict[str, torch.Tensor]) -> str:
    d = tempfile.mkdtemp(prefix="me_logozen_")
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file({k: v.contiguous() for k, v in weights.items()}, os.path.join(d, "model.safetensors"))
    return d


@functools.lru_cache(maxsize=None)
def folder(name: str) -> str:
    cfg, seed, _ = ALL[name]
    return write_folder(cfg, tensors(cfg, seed))
