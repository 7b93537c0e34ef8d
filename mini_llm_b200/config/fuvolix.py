"""Configuration of Fuvolix: a stack whose layers each name their mixer.

``config.json`` is nested: ``vocab``, ``width``, ``norm`` (``eps``, ``groups``), ``canon``
(``taps``: the short convolution in front of every mixer) and ``layers``, a list whose entries
give ``type`` (which mixer), ``mixer`` (its sizes and constants) and ``mlp`` (``kind``, ``ff``; or
null for a layer without feed-forward).  Every size and constant is read from there; a missing
or ill-typed key is an error that names its path.
"""

from __future__ import annotations

from dataclasses import dataclass, field

from .base import ConfigError, ModelConfig, _typed

MIXER_KEYS = {
    "latent_attention": {"heads": int, "dim": int, "rot_dim": int, "vdim": int, "kv_rank": int, "scale": float},
    "mlstm": {"heads": int, "dim": int, "vdim": int, "gate_cap": float},
    "lightning": {"heads": int, "dim": int, "vdim": int},
}
MLP_KINDS = ("dense",)


def _section(raw, key, where=""):
    value = raw.get(key)
    if not isinstance(value, dict):
        raise ConfigError(f"config key '{where}{key}': expected an object, got {value!r}")
    return value


def _take(raw, key, kind, where):
    if key not in raw or raw[key] is None:
        raise ConfigError(f"config key '{where}{key}' is missing")
    return _typed(f"{where}{key}", raw[key], kind)


def _positive(value, key):
    if value <= 0:
        raise ConfigError(f"config key '{key}': must be positive, got {value!r}")
    return value


def read_layer(raw, index: int) -> dict:
    """One entry of ``layers``, checked and typed."""
    where = f"layers[{index}]."
    if not isinstance(raw, dict):
        raise ConfigError(f"config key 'layers[{index}]': expected an object, got {raw!r}")
    kind = _take(raw, "type", str, where)
    if kind not in MIXER_KEYS:
        raise ConfigError(f"config key '{where}type': unknown mixer '{kind}' (known: {', '.join(sorted(MIXER_KEYS))})")
    given = _section(raw, "mixer", where)
    mixer = {}
    for key, typ in MIXER_KEYS[kind].items():
        mixer[key] = _take(given, key, typ, where + "mixer.")
        if key != "scale":
            _positive(mixer[key], where + "mixer." + key)
    if kind == "latent_attention":
        rot = _section(given, "rot", where + "mixer.")
        mixer["rot"] = {"base": _positive(_take(rot, "base", float, where + "mixer.rot."), where + "mixer.rot.base"),
                        "dims": _take(rot, "dims", int, where + "mixer.rot.")}
        if mixer["rot"]["dims"] % 2 or not 0 <= mixer["rot"]["dims"] <= mixer["rot_dim"]:
            raise ConfigError(f"config key '{where}mixer.rot.dims': an even number of at most rot_dim = "
                              f"{mixer['rot_dim']} dimensions is rotated, got {mixer['rot']['dims']}")
    if kind == "lightning":
        decay = given.get("decay")
        if not isinstance(decay, list) or len(decay) != mixer["heads"]:
            raise ConfigError(f"config key '{where}mixer.decay': expected {mixer['heads']} numbers (one per head), got {decay!r}")
        mixer["decay"] = [_typed(f"{where}mixer.decay[{h}]", d, float) for h, d in enumerate(decay)]
    mlp = raw.get("mlp")
    if mlp is not None:
        if not isinstance(mlp, dict):
            raise ConfigError(f"config key '{where}mlp': expected an object or null, got {mlp!r}")
        kind_ff = _take(mlp, "kind", str, where + "mlp.")
        if kind_ff not in MLP_KINDS:
            raise ConfigError(f"config key '{where}mlp.kind': unknown feed-forward '{kind_ff}' (known: {', '.join(MLP_KINDS)})")
        mlp = {"kind": kind_ff, "ff": _positive(_take(mlp, "ff", int, where + "mlp."), where + "mlp.ff")}
    return {"type": kind, "mixer": mixer, "mlp": mlp}


@dataclass(frozen=True)
class FuvolixConfig(ModelConfig):
    vocab: int = field(default=0, metadata={"kind": int})
    width: int = field(default=0, metadata={"kind": int})
    norm_eps: float = field(default=0.0, metadata={"kind": float})
    norm_groups: int = field(default=1, metadata={"kind": int})
    canon_taps: int = field(default=1, metadata={"kind": int})
    layers: tuple = ()

    @classmethod
    def from_dict(cls, raw: dict, architecture: str | None = None) -> "FuvolixConfig":
        if not isinstance(raw, dict):
            raise ConfigError("config.json must hold a JSON object")
        norm, canon = _section(raw, "norm"), _section(raw, "canon")
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError(f"config key 'layers': expected a list of layers, got {layers!r}")
        return cls(architecture=architecture or raw.get("architecture") or "Fuvolix",
                   vocab=_positive(_take(raw, "vocab", int, ""), "vocab"),
                   width=_positive(_take(raw, "width", int, ""), "width"),
                   norm_eps=_take(norm, "eps", float, "norm."),
                   norm_groups=_positive(_take(norm, "groups", int, "norm."), "norm.groups"),
                   canon_taps=_positive(_take(canon, "taps", int, "canon."), "canon.taps"),
                   layers=tuple(read_layer(layer, index) for index, layer in enumerate(layers)))

    def __post_init__(self):
        if self.width % self.norm_groups != 0:
            raise ConfigError(f"config key 'norm.groups': a width of {self.width} does not split into "
                              f"{self.norm_groups} equal groups")

    def to_dict(self) -> dict:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.norm_eps, "groups": self.norm_groups}, "canon": {"taps": self.canon_taps},
                "layers": [dict(layer) for layer in self.layers]}
