"""Gevulorn as a plan of parts.

Every layer is a block whose mixer and feed-forward read the same residual stream side by side (``parallel``) through
layer norms with weight and bias.  The mixer is gated linear attention (``gla``) or grouped-query attention with a learned
sink (``masked_sink_attention``) in one of two forms: plain projections, rotation, then a weightless norm of q and k, a
window that keeps the first tokens; or biased projections, a weighted norm of q and k in front of a rotation with rescaled
frequencies, capped scores and chunks.  The feed-forward is W_down relu(W_up h)^2 (``activation_mlp``) or routed
SiLU-gated experts with a shared one (``routed_experts``).  A range of layers may run several times in a row with the same
weights: every pass has cache slots of its own and adds its own vector to the stream in front of its first layer.  The
logits are capped.  Layer i's tensors are ``l<i>.*``; all numbers come from the configuration.
"""
from __future__ import annotations

from ..config.model_config import ConfigError, GevulornConfig
from ..config.registry import Architecture, register_architecture
from ..parts import BlockSpec, LayerCall, ModelPlan, PartSpec, SharedRef


def _rotation(m: dict, shared: dict):
    rot = m.get("rot")
    if not rot or not rot["dims"]:
        return None
    sc = rot.get("scaling")
    key = f"rot_{rot['dims']}_{rot['base']!r}_{sorted(sc.items()) if sc else None}"      # layers with the same rotation share one object
    shared.setdefault(key, PartSpec("rope_frequencies", {"rotary_dim": rot["dims"], "theta": rot["base"], "scaling": sc}))
    return SharedRef(key)


def gevulorn_plan(cfg: GevulornConfig) -> ModelPlan:
    W, eps = cfg.hidden_size, cfg.norm_eps
    blocks, shared = [], {}
    for i, layer in enumerate(cfg.layers):
        m, kind = layer["mixer"], layer["type"]
        if kind == "gla":
            if "decay_rank" not in m:
                raise ConfigError(f"layer {i}: the rank of the decay's projection is unknown (read it from the weights: "
                                  f"the shape of l{i}.mix.a1)")
            mixer = PartSpec("gla", {"hidden_size": W, "num_heads": m["heads"], "dim": m["dim"], "vdim": m["vdim"],
                                     "decay_rank": m["decay_rank"], "tau": m["tau"], "norm_eps": eps})
        else:
            mask = m.get("mask")
            args = {"hidden_size": W, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "dim": m["dim"], "vdim": m["vdim"],
                    "scale": m["scale"], "norm_eps": eps, "position_encoding": _rotation(m, shared), "sink": True}
            if kind == "attention":
                args.update(qk_norm="after", bias=False, softcap=m.get("softcap"),
                            mask=("window", mask["size"], mask.get("keep_first", 0)) if mask else None)
            else:
                args.update(qk_norm="before", bias=True, softcap=m.get("softcap"), mask=("chunk", mask["size"]) if mask else None)
            mixer = PartSpec("masked_sink_attention", args)
        mlp, ffn = layer["mlp"], None
        if mlp is not None and mlp["kind"] == "dense":
            ffn = PartSpec("activation_mlp", {"hidden_size": W, "intermediate_size": mlp["ff"], "activation": "relu_squared"})
        elif mlp is not None:
            silu_gated = {"limit": None, "alpha": 1.0, "shift": 0.0}
            ffn = PartSpec("routed_experts", {
                "hidden_size": W, "num_experts": mlp["router"]["experts"], "top": mlp["router"]["top"],
                "expert_size": mlp["expert"]["ff"], "router_bias": False, **silu_gated,
                "shared": {"intermediate_size": mlp["shared"]["ff"], **silu_gated} if mlp.get("shared") else None})
        blocks.append(BlockSpec(mixer=mixer, feed_forward=ffn, kind="parallel",
                                mixer_norm=PartSpec("layernorm", {"size": W, "eps": eps, "param": "norm1", "bias": "norm1.b"}),
                                feed_forward_norm=PartSpec("layernorm", {"size": W, "eps": eps, "param": "norm2", "bias": "norm2.b"}),
                                mixer_prefix="mix.", feed_forward_prefix="mlp.", mixer_norm_prefix="", feed_forward_norm_prefix=""))
    # every run of a layer has a cache slot of its own: a looped layer keeps one cache or state per pass
    schedule = [LayerCall(i, slot, True, add_row=t) for slot, (i, t) in enumerate(cfg.layer_runs())]
    return ModelPlan(
        vocab_size=cfg.vocab_size, hidden_size=W, blocks=blocks, schedule=schedule,
        final_norm=PartSpec("layernorm", {"size": W, "eps": eps, "param": "final.norm", "bias": "final.norm.b"}),
        tie_word_embeddings=False, max_position=cfg.max_position_embeddings, shared=shared,
        embed_prefix="", block_prefix="l{i}.", final_norm_prefix="", head_prefix="", embed_param="embed", head_param="head",
        embedding_scale=cfg.embedding_scale, logit_softcap=cfg.logit_softcap,
        pass_vectors=("loop.step", cfg.loop["times"]) if cfg.loop else None)


register_architecture(Architecture("Gevulorn", GevulornConfig.from_dict, gevulorn_plan), replace=True)
