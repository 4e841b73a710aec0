"""Logozen as a plan of parts.

Every layer is a hyper-connection block (several residual streams, a layer norm and a short causal convolution in
front of each sub-layer) around one of two mixers, attention through a latent with a sink and a gate per head, or an
mLSTM recurrence, and an optional dense PolyNorm feed-forward.  The embedding is scaled; the last norm reads the sum
of the streams.  Layer i's tensors are ``l<i>.*``; all numbers come from the configuration.
"""
from __future__ import annotations

from ..config.model_config import LogozenConfig
from ..config.registry import Architecture, register_architecture
from ..parts import BlockSpec, LayerCall, ModelPlan, PartSpec, SharedRef


def logozen_plan(cfg: LogozenConfig) -> ModelPlan:
    W, eps = cfg.hidden_size, cfg.norm_eps
    blocks, shared = [], {}
    for layer in cfg.layers:
        m = layer["mixer"]
        if layer["type"] == "latent_attention":
            key = f"rot_{m['rot']['dims']}_{m['rot']['base']!r}"          # layers with the same rotation share one object
            shared.setdefault(key, PartSpec("rope_interleaved", {"rotary_dim": m["rot"]["dims"], "theta": m["rot"]["base"]}))
            mixer = PartSpec("latent_attention", {
                "hidden_size": W, "num_heads": m["heads"], "dim": m["dim"], "rot_dim": m["rot_dim"], "vdim": m["vdim"],
                "kv_rank": m["kv_rank"], "scale": m["scale"], "norm_eps": eps, "position_encoding": SharedRef(key)})
        else:
            mixer = PartSpec("mlstm", {"hidden_size": W, "num_heads": m["heads"], "dim": m["dim"], "vdim": m["vdim"],
                                       "gate_cap": m["gate_cap"], "norm_eps": eps})
        ffn = None
        if layer["mlp"] is not None:
            ffn = PartSpec("polynorm_mlp", {"hidden_size": W, "intermediate_size": layer["mlp"]["ff"], "eps": eps})
        blocks.append(BlockSpec(
            mixer=mixer, feed_forward=ffn, kind="hyper_connection",
            mixer_norm=PartSpec("layernorm", {"size": W, "eps": eps, "streams": cfg.streams, "param": "norm1"}),
            feed_forward_norm=PartSpec("layernorm", {"size": W, "eps": eps, "streams": cfg.streams, "param": "norm2"}),
            mixer_prefix="mix.", feed_forward_prefix="mlp.", mixer_norm_prefix="", feed_forward_norm_prefix="",
            args={"streams": cfg.streams, "width": W, "taps": cfg.canon_taps}))
    n = len(blocks)
    return ModelPlan(
        vocab_size=cfg.vocab_size, hidden_size=W, blocks=blocks, schedule=[LayerCall(i, i, True) for i in range(n)],
        final_norm=PartSpec("layernorm", {"size": W, "eps": eps, "streams": cfg.streams, "param": "final.norm"}),
        tie_word_embeddings=False, max_position=cfg.max_position_embeddings, shared=shared,
        embed_prefix="", block_prefix="l{i}.", final_norm_prefix="", head_prefix="",
        embed_param="embed", head_param="head", embedding_scale=cfg.embedding_scale, streams=cfg.streams)


register_architecture(Architecture("Logozen", LogozenConfig.from_dict, logozen_plan), replace=True)
