"""Galupel as a plan of parts.

Every layer is a block whose norms sit behind its sub-layers (``post_norm``): x <- x + norm1(mixer(x)), then
x <- x + norm2(ff(x)), RMS norms in groups (``group_rmsnorm``); the sub-layers read the stream itself.  The mixer is
grouped-query attention without positions over a window and pooled blocks of tokens behind it
(``pooled_window_attention``; a layer may read an earlier layer's keys and values, ``kv_from``, with its own queries, window
and block size) or attention through a latent with a rotated part and a window (``latent_attention``).  The feed-forward is a
mixture of small experts W_down gelu(W_up h), routed by sigmoid scores with a correction over groups of experts
(``routed_experts`` with ``routing="sigmoid_groups"``), or absent.  The embedding passes through a norm, is also the output
matrix, and the logits are scaled and capped.  Layer i's tensors are ``l<i>.*``; all numbers come from the configuration.
"""
from __future__ import annotations

from ..config.model_config import GalupelConfig
from ..config.registry import Architecture, register_architecture
from ..parts import BlockSpec, LayerCall, ModelPlan, PartSpec, SharedRef


def galupel_plan(cfg: GalupelConfig) -> ModelPlan:
    W, eps = cfg.hidden_size, cfg.norm_eps

    def norm(name: str) -> PartSpec:
        return PartSpec("group_rmsnorm", {"size": W, "eps": eps, "groups": cfg.norm_groups, "param": name})
    # What the token pages of a layer with keys and values of its own must keep: the widest window, and the longest block
    # (a block's means are formed when its last token arrives), among the layers that read them.
    keep: dict[int, int] = {}
    for i, layer in enumerate(cfg.layers):
        if layer["type"] == "attention":
            m = layer["mixer"]
            src = m.get("kv_from", i)
            keep[src] = max(keep.get(src, 1), m["mask"]["size"], m["mask"].get("pool", 1))
    blocks, shared, schedule = [], {}, []
    for i, layer in enumerate(cfg.layers):
        m = layer["mixer"]
        src = i
        if layer["type"] == "attention":
            src = m.get("kv_from", i)
            mixer = PartSpec("pooled_window_attention", {
                "hidden_size": W, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "dim": m["dim"], "vdim": m["vdim"],
                "scale": m["scale"], "norm_eps": eps, "window": m["mask"]["size"], "pool": m["mask"].get("pool"),
                "cache_window": keep[src], "own_kv": src == i, "head_scale": True, "out_dtype": "float32"})
        else:
            rope = None
            if m.get("rot") and m["rot"]["dims"]:
                key = f"rot_{m['rot']['dims']}_{m['rot']['base']!r}"          # layers with the same rotation share one object
                shared.setdefault(key, PartSpec("rope_interleaved", {"rotary_dim": m["rot"]["dims"], "theta": m["rot"]["base"]}))
                rope = SharedRef(key)
            mixer = PartSpec("latent_attention", {
                "hidden_size": W, "num_heads": m["heads"], "dim": m["dim"], "rot_dim": m["rot_dim"], "vdim": m["vdim"],
                "kv_rank": m["kv_rank"], "scale": m["scale"], "norm_eps": eps, "position_encoding": rope, "sink": False,
                "gate": False, "window": m["mask"]["size"] if m.get("mask") else None, "out_dtype": "float32"})
        mlp, ffn = layer["mlp"], None
        if mlp is not None:
            r = mlp["router"]
            ffn = PartSpec("routed_experts", {
                "hidden_size": W, "num_experts": r["experts"], "top": r["top"], "expert_size": mlp["expert"]["ff"],
                "router_bias": False, "routing": "sigmoid_groups", "groups": (r["groups"]["count"], r["groups"]["keep"]),
                "correction": True, "activation": "gelu", "out_dtype": "float32"})
        blocks.append(BlockSpec(mixer=mixer, feed_forward=ffn, kind="post_norm", mixer_norm=norm("norm1"),
                                feed_forward_norm=norm("norm2"), mixer_prefix="mix.", feed_forward_prefix="mlp.",
                                mixer_norm_prefix="", feed_forward_norm_prefix=""))
        schedule.append(LayerCall(i, i, True, kv_slot=src if src != i else None))
    return ModelPlan(
        vocab_size=cfg.vocab_size, hidden_size=W, blocks=blocks, schedule=schedule, final_norm=norm("final.norm"),
        tie_word_embeddings=True, max_position=cfg.max_position_embeddings, shared=shared,
        embed_prefix="", block_prefix="l{i}.", final_norm_prefix="", head_prefix="", embed_param="embed", head_param="head",
        embed_norm=norm("embed.norm"), logit_scale=cfg.logit_scale, logit_softcap=cfg.logit_softcap)


register_architecture(Architecture("Galupel", GalupelConfig.from_dict, galupel_plan), replace=True)
