"""Configuration of Sumozen: a stack whose layers each name their mixer and carry a routed feed-forward.

``config.json`` is nested: ``vocab``, ``width``, ``norm`` (``eps``) and ``layers``, a list whose
entries give ``type`` ("parallel": a softmax attention and a gated delta rule side by side;
"mamba2": a state-space mixer), ``mixer`` (its sizes and constants) and ``mlp`` (``kind`` "moe" with
``router``, ``expert`` and an optional ``shared`` expert; or null for a layer without feed-forward).
Every size and constant is read from there; a missing or ill-typed key is an error that names
its path.
"""

from __future__ import annotations

from dataclasses import dataclass, field

from .base import ConfigError, ModelConfig, _typed

LEFT_KEYS = {"heads": int, "kv_heads": int, "dim": int, "vdim": int, "conv": int, "scale": float}
RIGHT_KEYS = {"heads": int, "kv_heads": int, "dim": int, "vdim": int, "conv": int}
MAMBA_KEYS = {"heads": int, "vdim": int, "state": int, "groups": int, "norm_groups": int, "conv": int}
SCALING_KEYS = ("factor", "original", "fast", "slow")


def _section(raw, key, where=""):
    value = raw.get(key) if isinstance(raw, dict) else None
    if not isinstance(value, dict):
        raise ConfigError(f"config key '{where}{key}': expected an object, got {value!r}")
    return value


def _take(raw, key, kind, where, positive=True):
    if key not in raw or raw[key] is None:
        raise ConfigError(f"config key '{where}{key}' is missing")
    value = _typed(f"{where}{key}", raw[key], kind)
    if positive and value <= 0:
        raise ConfigError(f"config key '{where}{key}': must be positive, got {value!r}")
    return value


def _sizes(raw, keys, where):
    return {key: _take(raw, key, kind, where) for key, kind in keys.items()}


def _multiple(sizes, many, few, where):
    if sizes[many] % sizes[few] != 0:
        raise ConfigError(f"config key '{where}{many}': {sizes[many]} is not a multiple of {few} = {sizes[few]}")


def read_rotation(raw, where, dim):
    rot = {"base": _take(raw, "base", float, where), "dims": _take(raw, "dims", int, where, positive=False)}
    if rot["base"] <= 1.0:
        raise ConfigError(f"config key '{where}base': must be larger than 1, got {rot['base']!r}")
    if rot["dims"] < 0 or rot["dims"] % 2 or rot["dims"] > dim:
        raise ConfigError(f"config key '{where}dims': an even number of at most dim = {dim} entries is rotated, "
                          f"got {rot['dims']}")
    scaling = raw.get("scaling")
    if scaling is not None:
        if not isinstance(scaling, dict):
            raise ConfigError(f"config key '{where}scaling': expected an object or null, got {scaling!r}")
        rot["scaling"] = {key: _take(scaling, key, float, where + "scaling.") for key in SCALING_KEYS}
    else:
        rot["scaling"] = None
    return rot


def read_mixer(kind, raw, where):
    if kind == "parallel":
        left_raw, right_raw = _section(raw, "left", where), _section(raw, "right", where)
        left = _sizes(left_raw, LEFT_KEYS, where + "left.")
        _multiple(left, "heads", "kv_heads", where + "left.")
        left["rot"] = read_rotation(_section(left_raw, "rot", where + "left."), where + "left.rot.", left["dim"])
        cap = left_raw.get("softcap")
        left["softcap"] = _take(left_raw, "softcap", float, where + "left.") if cap is not None else None
        right = _sizes(right_raw, RIGHT_KEYS, where + "right.")
        _multiple(right, "heads", "kv_heads", where + "right.")
        return {"left": left, "right": right,
                "left_scale": _take(raw, "left_scale", float, where, positive=False),
                "right_scale": _take(raw, "right_scale", float, where, positive=False)}
    sizes = _sizes(raw, MAMBA_KEYS, where)
    _multiple(sizes, "heads", "groups", where)
    if (sizes["heads"] * sizes["vdim"]) % sizes["norm_groups"] != 0:
        raise ConfigError(f"config key '{where}norm_groups': {sizes['heads'] * sizes['vdim']} inner channels do not "
                          f"split into {sizes['norm_groups']} equal parts")
    return sizes


def read_mlp(raw, where):
    if raw is None:
        return None
    if not isinstance(raw, dict):
        raise ConfigError(f"config key '{where[:-1]}': expected an object or null, got {raw!r}")
    kind = _take(raw, "kind", str, where, positive=False)
    if kind != "moe":
        raise ConfigError(f"config key '{where}kind': unknown feed-forward '{kind}' (known: moe)")
    router = _section(raw, "router", where)
    mlp = {"kind": kind,
           "router": {"experts": _take(router, "experts", int, where + "router."), "top": _take(router, "top", int, where + "router.")},
           "expert": {"ff": _take(_section(raw, "expert", where), "ff", int, where + "expert.")}}
    if mlp["router"]["top"] > mlp["router"]["experts"]:
        raise ConfigError(f"config key '{where}router.top': {mlp['router']['top']} of {mlp['router']['experts']} experts")
    shared = raw.get("shared")
    if shared is not None:
        if not isinstance(shared, dict):
            raise ConfigError(f"config key '{where}shared': expected an object or null, got {shared!r}")
        mlp["shared"] = {"ff": _take(shared, "ff", int, where + "shared.")}
    else:
        mlp["shared"] = None
    return mlp


def read_layer(raw, index: int) -> dict:
    where = f"layers[{index}]."
    if not isinstance(raw, dict):
        raise ConfigError(f"config key 'layers[{index}]': expected an object, got {raw!r}")
    kind = _take(raw, "type", str, where, positive=False)
    if kind not in ("parallel", "mamba2"):
        raise ConfigError(f"config key '{where}type': unknown layer type '{kind}' (known: mamba2, parallel)")
    return {"type": kind, "mixer": read_mixer(kind, _section(raw, "mixer", where), where + "mixer."),
            "mlp": read_mlp(raw.get("mlp"), where + "mlp.")}


@dataclass(frozen=True)
class SumozenConfig(ModelConfig):
    vocab: int = field(default=0, metadata={"kind": int})
    width: int = field(default=0, metadata={"kind": int})
    norm_eps: float = field(default=0.0, metadata={"kind": float})
    layers: tuple = ()

    @classmethod
    def from_dict(cls, raw: dict, architecture: str | None = None) -> "SumozenConfig":
        if not isinstance(raw, dict):
            raise ConfigError("config.json must hold a JSON object")
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError(f"config key 'layers': expected a list of layers, got {layers!r}")
        return cls(architecture=architecture or raw.get("architecture") or "Sumozen",
                   vocab=_take(raw, "vocab", int, ""), width=_take(raw, "width", int, ""),
                   norm_eps=_take(_section(raw, "norm"), "eps", float, "norm.", positive=False),
                   layers=tuple(read_layer(layer, index) for index, layer in enumerate(layers)))

    def to_dict(self) -> dict:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
                "layers": [_plain(layer) for layer in self.layers]}


def _plain(value):
    if isinstance(value, dict):
        return {key: _plain(one) for key, one in value.items()}
    return value
