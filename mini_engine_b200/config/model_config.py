"""Typed model configuration read from an architecture's own ``config.json`` keys.

The reference reads the same keys through a ``transformers`` config object that it
uses duck-typed (config.py:25, models/qwen3.py:15-17,81-84,107-108).  Here the file
is parsed directly: every size and constant of the model comes from it, none is
written in code.  A key the engine cannot honour (an activation other than SiLU,
biased projections, scaled rotary embeddings) is refused with a clear error
instead of being ignored.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field, asdict
from typing import Any


class ConfigError(ValueError):
    """A config.json that is missing a key, or asks for what the engine does not do."""


def read_config_json(folder: str) -> dict[str, Any]:
    path = os.path.join(os.path.expanduser(folder), "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"no config.json in {folder!r}")
    with open(path) as f:
        raw = json.load(f)
    if not isinstance(raw, dict):
        raise ConfigError(f"{path}: top level must be a JSON object")
    return raw


def architecture_name(raw: dict[str, Any]) -> str:
    """``"architectures": [name]`` (the first entry), or ``"architecture": name``."""
    archs = raw.get("architectures")
    if isinstance(archs, list) and archs and isinstance(archs[0], str):
        return archs[0]
    if isinstance(raw.get("architecture"), str):
        return raw["architecture"]
    raise ConfigError("config.json has neither an 'architectures': [name] nor an 'architecture': name entry")


def _need(raw: dict, key: str, kind):
    if key not in raw or raw[key] is None:
        raise ConfigError(f"config.json lacks required key {key!r}")
    v = raw[key]
    if kind is int:
        if isinstance(v, bool) or not isinstance(v, int):
            raise ConfigError(f"config.json key {key!r} must be an integer, got {v!r}")
        return v
    if kind is float:
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"config.json key {key!r} must be a number, got {v!r}")
        return float(v)
    return v


@dataclass
class ModelConfig:
    """What every architecture's configuration offers to the engine."""

    architecture: str
    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    max_position_embeddings: int
    eos_token_id: int = -1

    def to_json_dict(self) -> dict[str, Any]:
        raise NotImplementedError


@dataclass
class Qwen3Config(ModelConfig):
    """Qwen3 dense decoder (models/qwen3.py:12-116 in the reference).

    ``head_dim`` is independent of ``hidden_size / num_attention_heads``
    (models/qwen3.py:17).  ``layer_types`` and ``sliding_window`` are config.json keys
    of this architecture that the reference never reads (all its layers attend to
    every key); here a layer whose type is ``"sliding_attention"`` attends to the last
    ``sliding_window`` keys, itself included, when ``use_sliding_window`` is true.
    """

    num_attention_heads: int = 0
    num_key_value_heads: int = 0
    head_dim: int = 0
    intermediate_size: int = 0
    rms_norm_eps: float = 0.0
    rope_theta: float = 0.0
    tie_word_embeddings: bool = False
    use_sliding_window: bool = False
    sliding_window: int | None = None
    layer_types: list[str] = field(default_factory=list)

    @classmethod
    def from_dict(cls, raw: dict[str, Any]) -> "Qwen3Config":
        H = _need(raw, "hidden_size", int)
        nh = _need(raw, "num_attention_heads", int)
        L = _need(raw, "num_hidden_layers", int)
        nkv = raw.get("num_key_value_heads")
        if nkv is None:
            nkv = nh
        hd = raw.get("head_dim")
        if hd is None:
            if H % nh:
                raise ConfigError(f"head_dim absent and hidden_size {H} is no multiple of {nh} heads")
            hd = H // nh
        # models/qwen3.py:81 reads rope_parameters["rope_theta"]; raw files carry it at top level.
        rope = raw.get("rope_parameters") or {}
        theta = rope.get("rope_theta", raw.get("rope_theta"))
        if theta is None:
            raise ConfigError("config.json lacks 'rope_theta' (top level or in 'rope_parameters')")
        scaling = raw.get("rope_scaling")
        rope_type = (scaling or {}).get("rope_type", (scaling or {}).get("type", rope.get("rope_type", "default")))
        if rope_type not in ("default", None):
            raise ConfigError(f"rope scaling {rope_type!r} is not supported (only plain rotary embeddings)")
        if raw.get("hidden_act", "silu") != "silu":
            raise ConfigError(f"hidden_act {raw['hidden_act']!r} is not supported (only 'silu')")
        if raw.get("attention_bias", False):
            raise ConfigError("attention_bias=true is not supported (projections are bias-free)")
        use_win = bool(raw.get("use_sliding_window", False))
        window = raw.get("sliding_window")
        layer_types = raw.get("layer_types")
        if use_win:
            if not isinstance(window, int) or window < 1:
                raise ConfigError(f"use_sliding_window needs a positive integer 'sliding_window', got {window!r}")
            if layer_types is None:
                first = raw.get("max_window_layers", L)
                layer_types = ["sliding_attention" if i >= first else "full_attention" for i in range(L)]
        else:
            layer_types = ["full_attention"] * L
        if len(layer_types) != L or any(t not in ("full_attention", "sliding_attention") for t in layer_types):
            raise ConfigError(f"layer_types must name {L} layers as full_attention or sliding_attention")
        eos = raw.get("eos_token_id", -1)
        if isinstance(eos, list):
            eos = eos[0] if eos else -1
        cfg = cls(
            architecture=architecture_name(raw),
            vocab_size=_need(raw, "vocab_size", int),
            hidden_size=H,
            num_hidden_layers=L,
            max_position_embeddings=_need(raw, "max_position_embeddings", int),
            eos_token_id=-1 if eos is None else int(eos),
            num_attention_heads=nh,
            num_key_value_heads=int(nkv),
            head_dim=int(hd),
            intermediate_size=_need(raw, "intermediate_size", int),
            rms_norm_eps=_need(raw, "rms_norm_eps", float),
            rope_theta=float(theta),
            tie_word_embeddings=bool(raw.get("tie_word_embeddings", False)),
            use_sliding_window=use_win,
            sliding_window=window if use_win else None,
            layer_types=list(layer_types),
        )
        cfg.validate()
        return cfg

    def validate(self) -> None:
        for name in ("vocab_size", "hidden_size", "num_hidden_layers", "max_position_embeddings",
                     "num_attention_heads", "num_key_value_heads", "head_dim", "intermediate_size"):
            if getattr(self, name) < 1:
                raise ConfigError(f"{name} must be positive, got {getattr(self, name)}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(f"{self.num_attention_heads} heads are no multiple of "
                              f"{self.num_key_value_heads} key/value heads")
        if self.head_dim % 2:
            raise ConfigError(f"head_dim {self.head_dim} must be even for rotary embeddings")
        if not self.rms_norm_eps > 0:
            raise ConfigError("rms_norm_eps must be positive")
        if not self.rope_theta > 0:
            raise ConfigError("rope_theta must be positive")

    def window_of_layer(self, i: int) -> int | None:
        return self.sliding_window if self.layer_types[i] == "sliding_attention" else None

    def to_json_dict(self) -> dict[str, Any]:
        d = asdict(self)
        arch = d.pop("architecture")
        d["architectures"] = [arch]
        d["hidden_act"] = "silu"
        d["attention_bias"] = False
        d["torch_dtype"] = "bfloat16"
        if not self.use_sliding_window:
            d.pop("layer_types")
        return d


_LOGOZEN_MIXERS = {
    "latent_attention": {"heads": int, "dim": int, "rot_dim": int, "vdim": int, "kv_rank": int, "scale": float},
    "mlstm": {"heads": int, "dim": int, "vdim": int, "gate_cap": float},
}


@dataclass
class LogozenConfig(ModelConfig):
    """Logozen: a decoder whose layers each name their mixer (attention through a latent, or an mLSTM recurrence) and an
    optional dense PolyNorm feed-forward, over several residual streams with a short convolution in front of every
    sub-layer.  config.json keys: ``vocab``, ``width``, ``streams``, ``embedding.scale``, ``norm.eps``, ``canon.taps``
    and ``layers``: a list of ``{"type", "mixer": {sizes and constants}, "mlp": {"kind": "dense", "ff"} | null}``.
    The design has no limit on positions; ``max_position_embeddings`` is what an int32 position allows the engine."""

    streams: int = 1
    embedding_scale: float = 1.0
    norm_eps: float = 0.0
    canon_taps: int = 1
    layers: list[dict[str, Any]] = field(default_factory=list)

    @classmethod
    def from_dict(cls, raw: dict[str, Any]) -> "LogozenConfig":
        def sub(key):
            v = raw.get(key)
            if not isinstance(v, dict):
                raise ConfigError(f"config.json lacks the object {key!r}")
            return v
        layers = _need(raw, "layers", list)
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json key 'layers' must be a list with at least one layer")
        checked = []
        for i, layer in enumerate(layers):
            if not isinstance(layer, dict) or layer.get("type") not in _LOGOZEN_MIXERS:
                raise ConfigError(f"layer {i}: 'type' must be one of {sorted(_LOGOZEN_MIXERS)}, got "
                                  f"{layer.get('type') if isinstance(layer, dict) else layer!r}")
            mixer = layer.get("mixer")
            if not isinstance(mixer, dict):
                raise ConfigError(f"layer {i}: lacks the object 'mixer'")
            m = {k: _need(mixer, k, kind) for k, kind in _LOGOZEN_MIXERS[layer["type"]].items()}
            if layer["type"] == "latent_attention":
                rot = mixer.get("rot")
                if not isinstance(rot, dict):
                    raise ConfigError(f"layer {i}: a latent_attention mixer lacks the object 'rot'")
                m["rot"] = {"base": _need(rot, "base", float), "dims": _need(rot, "dims", int)}
                if m["rot"]["dims"] % 2 or not 0 <= m["rot"]["dims"] <= m["rot_dim"]:
                    raise ConfigError(f"layer {i}: rot.dims {m['rot']['dims']} must be even and at most rot_dim {m['rot_dim']}")
                if not m["rot"]["base"] > 0:
                    raise ConfigError(f"layer {i}: rot.base must be positive")
            elif not m["gate_cap"] > 0:
                raise ConfigError(f"layer {i}: gate_cap must be positive")
            if any(v < 1 for k, v in m.items() if isinstance(v, int) and k != "rot_dim") or m.get("rot_dim", 0) < 0:
                raise ConfigError(f"layer {i}: the mixer's sizes must be positive: {m}")
            mlp = layer.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
                    raise ConfigError(f"layer {i}: 'mlp' must be null or of kind 'dense', got {mlp!r}")
                mlp = {"kind": "dense", "ff": _need(mlp, "ff", int)}
                if mlp["ff"] < 1:
                    raise ConfigError(f"layer {i}: mlp.ff must be positive")
            checked.append({"type": layer["type"], "mixer": m, "mlp": mlp})
        eos = raw.get("eos_token_id", -1)
        cfg = cls(architecture=architecture_name(raw), vocab_size=_need(raw, "vocab", int), hidden_size=_need(raw, "width", int),
                  num_hidden_layers=len(checked), max_position_embeddings=int(raw.get("max_position_embeddings", 1 << 30)),
                  eos_token_id=-1 if eos is None else int(eos), streams=int(raw.get("streams", 1)),
                  embedding_scale=_need(sub("embedding"), "scale", float), norm_eps=_need(sub("norm"), "eps", float),
                  canon_taps=_need(sub("canon"), "taps", int), layers=checked)
        for name in ("vocab_size", "hidden_size", "streams", "canon_taps"):
            if getattr(cfg, name) < 1:
                raise ConfigError(f"{name} must be positive, got {getattr(cfg, name)}")
        if cfg.streams > 16:
            raise ConfigError(f"{cfg.streams} residual streams are not supported (up to 16)")
        if not cfg.norm_eps > 0:
            raise ConfigError("norm.eps must be positive")
        return cfg

    def to_json_dict(self) -> dict[str, Any]:
        return {"architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size, "streams": self.streams,
                "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps}, "canon": {"taps": self.canon_taps},
                "layers": self.layers}


def _opt_object(raw: dict, key: str, where: str):
    v = raw.get(key)
    if v is not None and not isinstance(v, dict):
        raise ConfigError(f"{where}: {key!r} must be an object or absent, got {v!r}")
    return v


def _glu_sizes(raw: dict, where: str) -> dict[str, Any]:
    out = {"ff": _need(raw, "ff", int)}
    if out["ff"] < 1:
        raise ConfigError(f"{where}: ff must be positive")
    if raw.get("limit") is not None:
        out["limit"] = _need(raw, "limit", float)
        if not out["limit"] > 0:
            raise ConfigError(f"{where}: limit must be positive")
    return out


@dataclass
class PugadraConfig(ModelConfig):
    """Pugadra: a decoder of attention layers whose sub-layers are normalised on both sides and scaled by
    ``residual_mult`` before they join the residual stream, with a per-layer input from the token itself behind the
    feed-forward.  config.json keys: ``vocab``, ``width``, ``norm.eps``, ``residual_mult``, ``token_side.dim`` (absent: no
    token input) and ``layers``: a list of ``{"type": "attention", "mixer": {heads, kv_heads, dim, vdim, scale, conv (taps),
    rot {base, dims}, mask {size}, kv_from}, "mlp": dense {ff, limit} | moe {router {experts, top}, expert {ff, limit},
    shared {ff, limit}} | null}``.  ``conv``, ``rot``, ``mask``, ``kv_from``, ``shared`` and every ``limit`` may be absent.
    The embedding is also the output matrix.  The design has no limit on positions; ``max_position_embeddings`` is what
    an int32 position allows the engine."""

    norm_eps: float = 0.0
    residual_mult: float = 1.0
    side_dim: int = 0
    layers: list[dict[str, Any]] = field(default_factory=list)

    @classmethod
    def from_dict(cls, raw: dict[str, Any]) -> "PugadraConfig":
        layers = _need(raw, "layers", list)
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json key 'layers' must be a list with at least one layer")
        checked = []
        for i, layer in enumerate(layers):
            where = f"layer {i}"
            if not isinstance(layer, dict) or layer.get("type") != "attention":
                raise ConfigError(f"{where}: 'type' must be 'attention', got {layer.get('type') if isinstance(layer, dict) else layer!r}")
            mixer = layer.get("mixer")
            if not isinstance(mixer, dict):
                raise ConfigError(f"{where}: lacks the object 'mixer'")
            m: dict[str, Any] = {k: _need(mixer, k, int) for k in ("heads", "kv_heads", "dim", "vdim")}
            m["scale"] = _need(mixer, "scale", float)
            if any(m[k] < 1 for k in ("heads", "kv_heads", "dim", "vdim")) or m["heads"] % m["kv_heads"]:
                raise ConfigError(f"{where}: sizes must be positive and heads a multiple of kv_heads: {m}")
            if mixer.get("conv") is not None:
                m["conv"] = _need(mixer, "conv", int)
                if m["conv"] < 1:
                    raise ConfigError(f"{where}: conv must be a positive number of taps")
            rot = _opt_object(mixer, "rot", where)
            if rot is not None:
                m["rot"] = {"base": _need(rot, "base", float), "dims": _need(rot, "dims", int)}
                if m["rot"]["dims"] % 2 or not 0 <= m["rot"]["dims"] <= m["dim"] or not m["rot"]["base"] > 0:
                    raise ConfigError(f"{where}: rot.dims must be even and at most dim, rot.base positive: {m['rot']}")
                if m["rot"]["dims"] and m["dim"] % 2:
                    raise ConfigError(f"{where}: a rotated head needs an even dim, got {m['dim']}")
            mask = _opt_object(mixer, "mask", where)
            if mask is not None and mask.get("size") is not None:
                m["mask"] = {"size": _need(mask, "size", int)}
                if m["mask"]["size"] < 1:
                    raise ConfigError(f"{where}: mask.size must be positive")
            if mixer.get("kv_from") is not None:
                j = m["kv_from"] = _need(mixer, "kv_from", int)
                if not 0 <= j < i or "kv_from" in checked[j]["mixer"]:
                    raise ConfigError(f"{where}: kv_from must name an earlier layer with keys and values of its own, got {j}")
                src = checked[j]["mixer"]
                if any(src[k] != m[k] for k in ("kv_heads", "dim", "vdim")) or src.get("rot") != m.get("rot"):
                    raise ConfigError(f"{where}: layer {j}'s key/value heads, sizes and rotation differ from this layer's")
            mlp = layer.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") not in ("dense", "moe"):
                    raise ConfigError(f"{where}: 'mlp' must be null or of kind 'dense' or 'moe', got {mlp!r}")
                if mlp["kind"] == "dense":
                    mlp = {"kind": "dense", **_glu_sizes(mlp, where + " mlp")}
                else:
                    router, expert = mlp.get("router"), mlp.get("expert")
                    if not isinstance(router, dict) or not isinstance(expert, dict):
                        raise ConfigError(f"{where}: a moe feed-forward needs the objects 'router' and 'expert'")
                    out = {"kind": "moe", "router": {"experts": _need(router, "experts", int), "top": _need(router, "top", int)},
                           "expert": _glu_sizes(expert, where + " mlp.expert")}
                    if not 1 <= out["router"]["top"] <= out["router"]["experts"]:
                        raise ConfigError(f"{where}: router.top must lie between 1 and router.experts")
                    shared = _opt_object(mlp, "shared", where)
                    if shared is not None:
                        out["shared"] = _glu_sizes(shared, where + " mlp.shared")
                    mlp = out
            checked.append({"type": "attention", "mixer": m, "mlp": mlp})
        norm = raw.get("norm")
        if not isinstance(norm, dict):
            raise ConfigError("config.json lacks the object 'norm'")
        side = _opt_object(raw, "token_side", "config.json")
        eos = raw.get("eos_token_id", -1)
        cfg = cls(architecture=architecture_name(raw), vocab_size=_need(raw, "vocab", int), hidden_size=_need(raw, "width", int),
                  num_hidden_layers=len(checked), max_position_embeddings=int(raw.get("max_position_embeddings", 1 << 30)),
                  eos_token_id=-1 if eos is None else int(eos), norm_eps=_need(norm, "eps", float),
                  residual_mult=float(raw.get("residual_mult", 1.0)), side_dim=_need(side, "dim", int) if side else 0, layers=checked)
        if cfg.vocab_size < 1 or cfg.hidden_size < 1 or cfg.side_dim < 0:
            raise ConfigError("vocab and width must be positive, token_side.dim not negative")
        if not cfg.norm_eps > 0:
            raise ConfigError("norm.eps must be positive")
        return cfg

    def to_json_dict(self) -> dict[str, Any]:
        d = {"architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size, "norm": {"eps": self.norm_eps},
             "residual_mult": self.residual_mult, "layers": self.layers}
        if self.side_dim:
            d["token_side"] = {"dim": self.side_dim}
        return d


def _positive_ints(raw: dict, keys, where: str) -> dict[str, int]:
    out = {k: _need(raw, k, int) for k in keys}
    if any(v < 1 for v in out.values()):
        raise ConfigError(f"{where}: sizes must be positive: {out}")
    return out


@dataclass
class GevulornConfig(ModelConfig):
    """Gevulorn: a decoder whose layers run their mixer and their feed-forward side by side on the same residual stream
    (x <- x + mixer(norm1(x)) + ff(norm2(x)), layer norms with weight and bias), and of which a range may run several
    times in a row with the same weights.  config.json keys: ``vocab``, ``width``, ``embedding.scale``, ``norm.eps``,
    ``logit_softcap`` (absent: none), ``loop`` {start, stop, times} (absent: every layer once) and ``layers``: a list of
    ``{"type", "mixer", "mlp"}`` with

    * type ``gla``: mixer {heads, dim, vdim, tau} (the rank of the decay's projection is the shape of its tensor's business:
      ``decay_rank``, absent: read from the weights by whoever has them);
    * type ``attention``: mixer {heads, kv_heads, dim, vdim, scale, rot {base, dims}, mask {size, keep_first}};
    * type ``attention_2``: mixer {heads, kv_heads, dim, vdim, scale, softcap, rot {base, dims, scaling {factor, low, high,
      original}}, mask {size}};
    * mlp: null, dense {ff} or moe {router {experts, top}, expert {ff}, shared {ff}}.

    ``rot``, ``mask``, ``keep_first``, ``scaling``, ``softcap`` and ``shared`` may be absent.  The design has no limit on
    positions; ``max_position_embeddings`` is what an int32 position allows the engine."""

    norm_eps: float = 0.0
    embedding_scale: float = 1.0
    logit_softcap: float | None = None
    loop: dict[str, int] | None = None
    layers: list[dict[str, Any]] = field(default_factory=list)

    @classmethod
    def from_dict(cls, raw: dict[str, Any]) -> "GevulornConfig":
        layers = _need(raw, "layers", list)
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json key 'layers' must be a list with at least one layer")
        checked = []
        for i, layer in enumerate(layers):
            where = f"layer {i}"
            kind = layer.get("type") if isinstance(layer, dict) else None
            if kind not in ("gla", "attention", "attention_2"):
                raise ConfigError(f"{where}: 'type' must be 'gla', 'attention' or 'attention_2', got {kind!r}")
            mixer = layer.get("mixer")
            if not isinstance(mixer, dict):
                raise ConfigError(f"{where}: lacks the object 'mixer'")
            if kind == "gla":
                m: dict[str, Any] = _positive_ints(mixer, ("heads", "dim", "vdim"), where)
                m["tau"] = _need(mixer, "tau", float)
                if not m["tau"] > 0:
                    raise ConfigError(f"{where}: tau must be positive")
                if mixer.get("decay_rank") is not None:
                    m.update(_positive_ints(mixer, ("decay_rank",), where))
            else:
                m = _positive_ints(mixer, ("heads", "kv_heads", "dim", "vdim"), where)
                if m["heads"] % m["kv_heads"]:
                    raise ConfigError(f"{where}: heads must be a multiple of kv_heads: {m}")
                m["scale"] = _need(mixer, "scale", float)
                rot = _opt_object(mixer, "rot", where)
                if rot is not None:
                    m["rot"] = {"base": _need(rot, "base", float), "dims": _need(rot, "dims", int)}
                    if m["rot"]["dims"] % 2 or not 0 <= m["rot"]["dims"] <= m["dim"] or not m["rot"]["base"] > 0:
                        raise ConfigError(f"{where}: rot.dims must be even and at most dim, rot.base positive: {m['rot']}")
                    sc = _opt_object(rot, "scaling", where)
                    if sc is not None:
                        m["rot"]["scaling"] = {k: _need(sc, k, float) for k in ("factor", "low", "high", "original")}
                        s = m["rot"]["scaling"]
                        if not (s["factor"] > 0 and s["original"] > 0 and s["high"] > s["low"] > 0):
                            raise ConfigError(f"{where}: rot.scaling needs factor > 0, original > 0 and high > low > 0: {s}")
                mask = _opt_object(mixer, "mask", where)
                if mask is not None and mask.get("size") is not None:
                    m["mask"] = {"size": _need(mask, "size", int)}
                    if m["mask"]["size"] < 1:
                        raise ConfigError(f"{where}: mask.size must be positive")
                    if mask.get("keep_first") is not None:
                        if kind != "attention":
                            raise ConfigError(f"{where}: only 'attention' keeps first tokens beside its window")
                        m["mask"]["keep_first"] = _need(mask, "keep_first", int)
                        if m["mask"]["keep_first"] < 0:
                            raise ConfigError(f"{where}: mask.keep_first must not be negative")
                if mixer.get("softcap") is not None:
                    m["softcap"] = _need(mixer, "softcap", float)
                    if not m["softcap"] > 0:
                        raise ConfigError(f"{where}: softcap must be positive")
            mlp = layer.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") not in ("dense", "moe"):
                    raise ConfigError(f"{where}: 'mlp' must be null or of kind 'dense' or 'moe', got {mlp!r}")
                if mlp["kind"] == "dense":
                    mlp = {"kind": "dense", **_positive_ints(mlp, ("ff",), where + " mlp")}
                else:
                    router, expert = mlp.get("router"), mlp.get("expert")
                    if not isinstance(router, dict) or not isinstance(expert, dict):
                        raise ConfigError(f"{where}: a moe feed-forward needs the objects 'router' and 'expert'")
                    out = {"kind": "moe", "router": _positive_ints(router, ("experts", "top"), where + " mlp.router"),
                           "expert": _positive_ints(expert, ("ff",), where + " mlp.expert")}
                    if out["router"]["top"] > out["router"]["experts"]:
                        raise ConfigError(f"{where}: router.top must lie between 1 and router.experts")
                    shared = _opt_object(mlp, "shared", where)
                    if shared is not None:
                        out["shared"] = _positive_ints(shared, ("ff",), where + " mlp.shared")
                    mlp = out
            checked.append({"type": kind, "mixer": m, "mlp": mlp})
        norm = raw.get("norm")
        if not isinstance(norm, dict):
            raise ConfigError("config.json lacks the object 'norm'")
        emb = _opt_object(raw, "embedding", "config.json")
        loop = _opt_object(raw, "loop", "config.json")
        if loop is not None:
            loop = {k: _need(loop, k, int) for k in ("start", "stop", "times")}
            if not 0 <= loop["start"] <= loop["stop"] <= len(checked) or loop["times"] < 1:
                raise ConfigError(f"loop must name a range of layers and a positive number of passes: {loop}")
            if loop["start"] == loop["stop"]:
                loop = None
        cap = raw.get("logit_softcap")
        eos = raw.get("eos_token_id", -1)
        cfg = cls(architecture=architecture_name(raw), vocab_size=_need(raw, "vocab", int), hidden_size=_need(raw, "width", int),
                  num_hidden_layers=len(checked), max_position_embeddings=int(raw.get("max_position_embeddings", 1 << 30)),
                  eos_token_id=-1 if eos is None else int(eos), norm_eps=_need(norm, "eps", float),
                  embedding_scale=_need(emb, "scale", float) if emb and emb.get("scale") is not None else 1.0,
                  logit_softcap=_need(raw, "logit_softcap", float) if cap is not None else None, loop=loop, layers=checked)
        if cfg.vocab_size < 1 or cfg.hidden_size < 1:
            raise ConfigError("vocab and width must be positive")
        if not cfg.norm_eps > 0:
            raise ConfigError("norm.eps must be positive")
        if cfg.logit_softcap is not None and not cfg.logit_softcap > 0:
            raise ConfigError("logit_softcap must be positive")
        return cfg

    def complete_from_tensor_shapes(self, shapes) -> None:
        """The rank of a gla layer's decay projection, where config.json does not give it, is the row count of the layer's
        ``mix.a1`` tensor.  ``shapes``: a callable that returns name -> shape (called only when something is missing)."""
        missing = [i for i, layer in enumerate(self.layers) if layer["type"] == "gla" and "decay_rank" not in layer["mixer"]]
        if not missing:
            return
        found = shapes()
        for i in missing:
            shape = found.get(f"l{i}.mix.a1")
            if shape is None or len(shape) != 2 or shape[0] < 1:
                raise ConfigError(f"layer {i}: neither config.json (decay_rank) nor the weights (l{i}.mix.a1) give the decay's rank")
            self.layers[i]["mixer"]["decay_rank"] = int(shape[0])

    def layer_runs(self) -> list[tuple[int, int | None]]:
        """The order in which layers run as (layer, pass) pairs: ``pass`` is the number of the pass for the first layer of
        every pass over the looped range (the pass's vector joins the stream there), else None."""
        n = len(self.layers)
        if not self.loop:
            return [(i, None) for i in range(n)]
        a, b, times = self.loop["start"], self.loop["stop"], self.loop["times"]
        runs: list[tuple[int, int | None]] = [(i, None) for i in range(a)]
        for t in range(times):
            runs += [(i, t if i == a else None) for i in range(a, b)]
        return runs + [(i, None) for i in range(b, n)]

    def to_json_dict(self) -> dict[str, Any]:
        d = {"architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size, "norm": {"eps": self.norm_eps},
             "embedding": {"scale": self.embedding_scale}, "layers": self.layers}
        if self.logit_softcap is not None:
            d["logit_softcap"] = self.logit_softcap
        if self.loop:
            d["loop"] = self.loop
        return d


@dataclass
class GalupelConfig(ModelConfig):
    """Galupel: a decoder whose sub-layers read the residual stream itself and join it through a norm of their OUTPUT,
    x <- x + norm1(mixer(x)), x <- x + norm2(ff(x)), with RMS norms taken over ``norm.groups`` equal parts of a row; the
    embedding passes through such a norm too, is also the output matrix, and the logits are scaled and capped.  config.json
    keys: ``vocab``, ``width``, ``norm`` {eps, groups}, ``logit_scale`` (absent: 1), ``logit_softcap`` (absent: none) and
    ``layers``: a list of ``{"type", "mixer", "mlp"}`` with

    * type ``attention``: mixer {heads, kv_heads, dim, vdim, scale, mask {size, pool}, kv_from}: grouped-query attention
      without positions over a window and pooled blocks of ``pool`` tokens behind it (``pool`` absent: the window alone);
      ``kv_from`` names an earlier layer of this type whose keys and values the layer reads with its own mask;
    * type ``latent_attention``: mixer {heads, dim, rot_dim, vdim, kv_rank, scale, rot {base, dims}, mask {size}}: attention
      through a latent with a rotated part and a window (``rot`` and ``mask`` may be absent);
    * mlp: null or moe {router {experts, top, groups {count, keep}}, expert {ff}} (``groups`` absent: one group).

    The design has no limit on positions; ``max_position_embeddings`` is what an int32 position allows the engine."""

    norm_eps: float = 0.0
    norm_groups: int = 1
    logit_scale: float = 1.0
    logit_softcap: float | None = None
    layers: list[dict[str, Any]] = field(default_factory=list)

    @classmethod
    def from_dict(cls, raw: dict[str, Any]) -> "GalupelConfig":
        layers = _need(raw, "layers", list)
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json key 'layers' must be a list with at least one layer")
        checked: list[dict[str, Any]] = []
        for i, layer in enumerate(layers):
            where = f"layer {i}"
            kind = layer.get("type") if isinstance(layer, dict) else None
            if kind not in ("attention", "latent_attention"):
                raise ConfigError(f"{where}: 'type' must be 'attention' or 'latent_attention', got {kind!r}")
            mixer = layer.get("mixer")
            if not isinstance(mixer, dict):
                raise ConfigError(f"{where}: lacks the object 'mixer'")
            mask = _opt_object(mixer, "mask", where)
            if kind == "attention":
                m: dict[str, Any] = _positive_ints(mixer, ("heads", "kv_heads", "dim", "vdim"), where)
                if m["heads"] % m["kv_heads"]:
                    raise ConfigError(f"{where}: heads must be a multiple of kv_heads: {m}")
                if mask is None or mask.get("size") is None:
                    raise ConfigError(f"{where}: an 'attention' layer needs mask.size")
                m["mask"] = _positive_ints(mask, ("size",), where + " mask")
                if mask.get("pool") is not None:
                    m["mask"].update(_positive_ints(mask, ("pool",), where + " mask"))
                if mixer.get("kv_from") is not None:
                    j = m["kv_from"] = _need(mixer, "kv_from", int)
                    if not 0 <= j < i or checked[j]["type"] != "attention" or "kv_from" in checked[j]["mixer"]:
                        raise ConfigError(f"{where}: kv_from must name an earlier 'attention' layer with keys and values of its own, got {j}")
                    src = checked[j]["mixer"]
                    if any(src[k] != m[k] for k in ("kv_heads", "dim", "vdim")):
                        raise ConfigError(f"{where}: layer {j}'s key/value heads and sizes differ from this layer's")
            else:
                m = _positive_ints(mixer, ("heads", "dim", "vdim", "kv_rank"), where)
                m["rot_dim"] = _need(mixer, "rot_dim", int)
                if m["rot_dim"] < 0:
                    raise ConfigError(f"{where}: rot_dim must not be negative")
                rot = _opt_object(mixer, "rot", where)
                if rot is not None:
                    m["rot"] = {"base": _need(rot, "base", float), "dims": _need(rot, "dims", int)}
                    if m["rot"]["dims"] % 2 or not 0 <= m["rot"]["dims"] <= m["rot_dim"] or not m["rot"]["base"] > 0:
                        raise ConfigError(f"{where}: rot.dims must be even and at most rot_dim, rot.base positive: {m['rot']}")
                if mask is not None and mask.get("size") is not None:
                    m["mask"] = _positive_ints(mask, ("size",), where + " mask")
            m["scale"] = _need(mixer, "scale", float)
            mlp = layer.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") != "moe":
                    raise ConfigError(f"{where}: 'mlp' must be null or of kind 'moe', got {mlp!r}")
                router, expert = mlp.get("router"), mlp.get("expert")
                if not isinstance(router, dict) or not isinstance(expert, dict):
                    raise ConfigError(f"{where}: a moe feed-forward needs the objects 'router' and 'expert'")
                r = _positive_ints(router, ("experts", "top"), where + " mlp.router")
                groups = _opt_object(router, "groups", where + " mlp.router")
                r["groups"] = _positive_ints(groups, ("count", "keep"), where + " mlp.router.groups") if groups else {"count": 1, "keep": 1}
                g = r["groups"]
                if r["experts"] % g["count"] or g["keep"] > g["count"] or g["keep"] * (r["experts"] // g["count"]) < r["top"]:
                    raise ConfigError(f"{where}: {g['keep']} of {g['count']} groups over {r['experts']} experts cannot give {r['top']} choices")
                mlp = {"kind": "moe", "router": r, "expert": _positive_ints(expert, ("ff",), where + " mlp.expert")}
            checked.append({"type": kind, "mixer": m, "mlp": mlp})
        norm = raw.get("norm")
        if not isinstance(norm, dict):
            raise ConfigError("config.json lacks the object 'norm'")
        cap = raw.get("logit_softcap")
        eos = raw.get("eos_token_id", -1)
        cfg = cls(architecture=architecture_name(raw), vocab_size=_need(raw, "vocab", int), hidden_size=_need(raw, "width", int),
                  num_hidden_layers=len(checked), max_position_embeddings=int(raw.get("max_position_embeddings", 1 << 30)),
                  eos_token_id=-1 if eos is None else int(eos), norm_eps=_need(norm, "eps", float),
                  norm_groups=_need(norm, "groups", int) if norm.get("groups") is not None else 1,
                  logit_scale=_need(raw, "logit_scale", float) if raw.get("logit_scale") is not None else 1.0,
                  logit_softcap=_need(raw, "logit_softcap", float) if cap is not None else None, layers=checked)
        if cfg.vocab_size < 1 or cfg.hidden_size < 1:
            raise ConfigError("vocab and width must be positive")
        if not cfg.norm_eps > 0:
            raise ConfigError("norm.eps must be positive")
        if cfg.norm_groups < 1 or cfg.hidden_size % cfg.norm_groups:
            raise ConfigError(f"norm.groups must divide width: {cfg.norm_groups} and {cfg.hidden_size}")
        if cfg.logit_softcap is not None and not cfg.logit_softcap > 0:
            raise ConfigError("logit_softcap must be positive")
        return cfg

    def to_json_dict(self) -> dict[str, Any]:
        d = {"architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size,
             "norm": {"eps": self.norm_eps, "groups": self.norm_groups}, "logit_scale": self.logit_scale, "layers": self.layers}
        if self.logit_softcap is not None:
            d["logit_softcap"] = self.logit_softcap
        return d
