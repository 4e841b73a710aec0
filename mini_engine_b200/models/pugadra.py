"""Pugadra as a plan of parts.

Every layer is a block with norms on both sides of its sub-layers (``sandwich_norm``) around grouped-query attention with
convolved, biased projections, a window, a sink of score 0 in the softmax and an output gate (``sink_attention``), a
clamped gated feed-forward, dense or routed with a shared expert, and a per-layer input from the token.  A layer may take
its keys and values from an earlier layer's cache (``kv_from``): it then has a cache slot of its own for its state only and
reads the other layer's pages.  The embedding is also the output matrix.  Layer i's tensors are ``l<i>.*``; all numbers
come from the configuration.
"""
from __future__ import annotations

from ..config.model_config import PugadraConfig
from ..config.registry import Architecture, register_architecture
from ..parts import BlockSpec, LayerCall, ModelPlan, PartSpec, SharedRef


def _glu_args(sizes: dict) -> dict:
    return {"intermediate_size": sizes["ff"], "limit": sizes.get("limit")}


def pugadra_plan(cfg: PugadraConfig) -> ModelPlan:
    W, eps = cfg.hidden_size, cfg.norm_eps
    n = len(cfg.layers)

    def norm(name: str) -> PartSpec:
        return PartSpec("rmsnorm", {"size": W, "eps": eps, "param": name, "unit_offset": True})
    # What the cache of a layer with keys and values of its own must keep: the widest window among its readers.
    keep: dict[int, list] = {}
    for i, layer in enumerate(cfg.layers):
        m = layer["mixer"]
        keep.setdefault(m.get("kv_from", i), []).append(m["mask"]["size"] if m.get("mask") else None)
    blocks, shared, schedule = [], {}, []
    for i, layer in enumerate(cfg.layers):
        m = layer["mixer"]
        rope = None
        if m.get("rot") and m["rot"]["dims"]:
            key = f"rot_{m['rot']['dims']}_{m['rot']['base']!r}"          # layers with the same rotation share one object
            shared.setdefault(key, PartSpec("rope_interleaved", {"rotary_dim": m["rot"]["dims"], "theta": m["rot"]["base"]}))
            rope = SharedRef(key)
        src = m.get("kv_from", i)
        windows = keep[src]
        mixer = PartSpec("sink_attention", {
            "hidden_size": W, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "dim": m["dim"], "vdim": m["vdim"],
            "scale": m["scale"], "position_encoding": rope, "window": m["mask"]["size"] if m.get("mask") else None,
            "cache_window": None if None in windows else max(windows), "conv_taps": m.get("conv"), "bias": True, "gate": True,
            "sink": True, "own_kv": src == i})
        mlp, ffn = layer["mlp"], None
        if mlp is not None and mlp["kind"] == "dense":
            ffn = PartSpec("clamped_glu", {"hidden_size": W, **_glu_args(mlp)})
        elif mlp is not None:
            ffn = PartSpec("routed_experts", {
                "hidden_size": W, "num_experts": mlp["router"]["experts"], "top": mlp["router"]["top"],
                "expert_size": mlp["expert"]["ff"], "limit": mlp["expert"].get("limit"), "router_bias": True,
                "shared": _glu_args(mlp["shared"]) if mlp.get("shared") else None})
        args = {"mult": cfg.residual_mult, "width": W, "post_mixer_norm": norm("norm1b"), "post_feed_forward_norm": norm("norm2b")}
        if cfg.side_dim:
            args["side"] = {"dim": cfg.side_dim, "first": i * cfg.side_dim, "table": SharedRef("token_side")}
        blocks.append(BlockSpec(mixer=mixer, feed_forward=ffn, kind="sandwich_norm", mixer_norm=norm("norm1"),
                                feed_forward_norm=norm("norm2"), mixer_prefix="mix.", feed_forward_prefix="mlp.",
                                mixer_norm_prefix="", feed_forward_norm_prefix="", args=args))
        schedule.append(LayerCall(i, i, True, kv_slot=src if src != i else None))
    return ModelPlan(
        vocab_size=cfg.vocab_size, hidden_size=W, blocks=blocks, schedule=schedule, final_norm=norm("final.norm"),
        tie_word_embeddings=True, max_position=cfg.max_position_embeddings, shared=shared,
        embed_prefix="", block_prefix="l{i}.", final_norm_prefix="", head_prefix="", embed_param="embed", head_param="head",
        tables={"token_side": ("side.embed", cfg.vocab_size, n * cfg.side_dim)} if cfg.side_dim else {})


register_architecture(Architecture("Pugadra", PugadraConfig.from_dict, pugadra_plan), replace=True)
