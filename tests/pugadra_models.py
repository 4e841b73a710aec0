"""Small Pugadra models for the tests: configurations that differ in every size and constant, and random weights.

The writer here knows the tensor names and shapes of the design by itself (it does not ask the engine), draws matrices
as N(0, gain / sqrt(inputs)) so that every layer changes the residual stream noticeably, and lets a test overwrite any
tensor before the folder is written.
"""
from __future__ import annotations

import functools
import json
import os
import tempfile

import torch
from safetensors.torch import save_file


def attn(heads, kv_heads, dim, vdim, conv=None, rot=None, base=10000.0, mask=None, kv_from=None, scale=None, mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": dim ** -0.5 if scale is None else scale}
    if conv is not None:
        m["conv"] = conv
    if rot is not None:
        m["rot"] = {"base": base, "dims": rot}
    if mask is not None:
        m["mask"] = {"size": mask}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m, "mlp": mlp}


def dense(ff, limit=None):
    return {"kind": "dense", "ff": ff, **({"limit": limit} if limit is not None else {})}


def moe(experts, top, ff, limit=None, shared=None):
    out = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff, **({"limit": limit} if limit is not None else {})}}
    if shared is not None:
        out["shared"] = {"ff": shared[0], **({"limit": shared[1]} if shared[1] is not None else {})}
    return out


def config(vocab, width, layers, eps=1e-5, mult=0.3, side=None):
    c = {"architecture": "Pugadra", "vocab": vocab, "width": width, "norm": {"eps": eps}, "residual_mult": mult, "layers": layers}
    if side:
        c["token_side"] = {"dim": side}
    return c


# A: two kv heads of four, keys of 16 and values of 24, half of a head rotated; a layer that takes another's keys with a
#    NARROWER window than the source's; a layer that sees every key and has no feed-forward; a router that takes one expert
A = config(101, 64, [
    attn(4, 2, 16, 24, conv=3, rot=8, base=5000.0, mask=40, mlp=dense(96, 1.5)),
    attn(4, 2, 16, 24, conv=3, rot=8, base=5000.0, mask=24, kv_from=0, mlp=moe(6, 2, 40, 2.0, shared=(48, 1.0))),
    attn(4, 4, 16, 8, conv=2, rot=16, mlp=None),
    attn(8, 4, 16, 8, conv=2, rot=16, mask=56, kv_from=2, scale=0.4, mlp=moe(4, 1, 32, 3.0)),
], eps=1e-6, mult=0.5, side=8)
# B: no size a multiple of 8; odd value sizes; windows that are no multiple of a page (of 8 tokens); four taps and one tap
#    (a weight and no state); a layer without rotation; feed-forwards without a limit; three of five experts; no token input
B = config(75, 52, [
    attn(3, 1, 10, 9, conv=4, rot=6, base=300.0, mask=33, mlp=dense(70)),
    attn(6, 3, 6, 5, conv=1, mask=17, mlp=moe(5, 3, 22)),
    attn(3, 1, 10, 9, conv=4, rot=6, base=300.0, mask=45, kv_from=0, mlp=dense(30, 0.7)),
], eps=2e-5, mult=1.0)
# C: heads of 64 and a window of 128 (the sizes the tensor-core kernels take), eight query heads on two kv heads, a sharing
#    layer with a WIDER window than its source, 16 experts
C = config(130, 128, [
    attn(8, 2, 64, 64, conv=3, rot=64, mask=96, mlp=dense(256, 2.0)),
    attn(8, 2, 64, 64, conv=3, rot=64, mask=128, kv_from=0, mlp=moe(16, 2, 64, 2.0, shared=(64, 2.0))),
    attn(4, 4, 32, 64, conv=2, rot=16, base=1e6, mlp=moe(8, 4, 48, 1.0)),
], eps=1e-5, mult=0.35, side=16)
# D: no convolution, as many kv heads as heads, a window of ONE token (a query sees itself and the sink), every expert chosen
D = config(64, 40, [
    attn(2, 2, 8, 8, rot=8, base=50.0, mask=1, mlp=moe(3, 3, 24, 2.0)),
    attn(5, 5, 8, 16, rot=4, base=50.0, mask=7, mlp=dense(56, 4.0)),
], eps=1e-5, mult=0.7, side=5)

ALL = {"A": (A, 1, 16), "B": (B, 2, 8), "C": (C, 3, 16), "D": (D, 4, 32)}        # config, seed, page size


def tensors(cfg: dict, seed: int, gain: float = 1.2) -> dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]
    side = cfg.get("token_side", {}).get("dim", 0)

    def mat(rows, cols, k=gain):
        return torch.randn(rows, cols, generator=g) * (k / cols ** 0.5)

    def around(n, mean, std):
        return mean + std * torch.randn(n, generator=g)

    def glu(prefix, ff):
        t[prefix + "gate"], t[prefix + "up"], t[prefix + "down"] = mat(ff, W, 1.6), mat(ff, W, 1.6), mat(W, ff, 1.0)
    t = {"embed": torch.randn(cfg["vocab"], W, generator=g) * 0.6, "final.norm": around(W, 0.0, 0.3)}
    if side:
        t["side.embed"] = torch.randn(cfg["vocab"], side * len(cfg["layers"]), generator=g)
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        H, G, Dk, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        t[p + "norm1"], t[p + "norm1b"] = around(W, 0.0, 0.3), around(W, 0.0, 0.3)
        pieces = [("q", H * Dk)] + ([("k", G * Dk), ("v", G * Dv)] if "kv_from" not in m else [])
        for name, n in pieces:
            t[p + "mix." + name] = mat(n, W, 1.5)
            t[p + "mix." + name + ".b"] = around(n, 0.0, 0.4)
            if "conv" in m:
                t[p + f"mix.{name}.conv"] = torch.randn(n, m["conv"], generator=g) * 0.6
        t[p + "mix.g"], t[p + "mix.o"] = mat(H * Dv, W, 1.5), mat(W, H * Dv, 1.2)
        mlp = layer["mlp"]
        if mlp is not None:
            t[p + "norm2"], t[p + "norm2b"] = around(W, 0.0, 0.3), around(W, 0.0, 0.3)
            if mlp["kind"] == "dense":
                glu(p + "mlp.", mlp["ff"])
            else:
                E = mlp["router"]["experts"]
                t[p + "mlp.router"], t[p + "mlp.router.b"] = mat(E, W, 2.0), around(E, 0.0, 0.5)
                for e in range(E):
                    glu(p + f"mlp.e{e}.", mlp["expert"]["ff"])
                if "shared" in mlp:
                    glu(p + "mlp.shared.", mlp["shared"]["ff"])
        if side:
            t[p + "side.gate"], t[p + "side.proj"], t[p + "side.norm"] = mat(side, W, 1.5), mat(W, side, 1.0), around(W, 1.0, 0.3)
    return {k: v.to(torch.bfloat16).contiguous() for k, v in t.items()}


def write_folder(cfg: dict, weights: dict[str, torch.Tensor]) -> str:
    d = tempfile.mkdtemp(prefix="me_pugadra_")
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file({k: v.contiguous() for k, v in weights.items()}, os.path.join(d, "model.safetensors"))
    return d


@functools.lru_cache(maxsize=None)
def folder(name: str) -> str:
    cfg, seed, _ = ALL[name]
    return write_folder(cfg, tensors(cfg, seed))
