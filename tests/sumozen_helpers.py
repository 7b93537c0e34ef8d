"""Shared by the Sumozen tests: small configurations (none with the sizes of any released model),
model folders with random weights that a test may then bend, and the plain logits."""

import json
import os

import numpy as np

import plain_sumozen as plain
from mini_llm_b200.config import config_from_dict, describe_model
from mini_llm_b200.weights.random_init import random_tensors
from mini_llm_b200.weights.safetensors_io import write_safetensors

YARN = {"factor": 4.0, "original": 64, "fast": 16.0, "slow": 2.0}


def moe(experts=5, top=2, ff=24, shared=40):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff},
            "shared": None if shared is None else {"ff": shared}}


def parallel(heads=4, kv_heads=2, dim=16, vdim=24, taps=3, rot_dims=12, base=300.0, scaling=YARN, scale=0.3, softcap=7.0,
             r_heads=4, r_kv_heads=2, r_dim=12, r_vdim=20, r_taps=4, left_scale=0.7, right_scale=1.2, mlp="default"):
    return {"type": "parallel",
            "mixer": {"left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": taps, "scale": scale,
                               "softcap": softcap, "rot": {"base": base, "dims": rot_dims, "scaling": scaling}},
                      "right": {"heads": r_heads, "kv_heads": r_kv_heads, "dim": r_dim, "vdim": r_vdim, "conv": r_taps},
                      "left_scale": left_scale, "right_scale": right_scale},
            "mlp": moe() if mlp == "default" else mlp}


def mamba(heads=4, vdim=12, state=20, groups=2, norm_groups=3, taps=4, mlp="default"):
    return {"type": "mamba2",
            "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "norm_groups": norm_groups, "conv": taps},
            "mlp": moe() if mlp == "default" else mlp}


def config(layers, width=96, vocab=211, eps=1e-5):
    return {"architecture": "Sumozen", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": list(layers)}


def full_stack(**kw):
    """Both layer types, with and without feed-forward, with other sizes in the second pair."""
    return config([parallel(), mamba(mlp=None),
                   parallel(heads=3, kv_heads=3, dim=8, vdim=8, taps=2, rot_dims=8, scaling=None, softcap=None, r_heads=2,
                            r_kv_heads=1, r_dim=20, r_vdim=8, r_taps=2, mlp=moe(experts=3, top=1, ff=16, shared=None)),
                   mamba(heads=2, vdim=24, state=8, groups=1, norm_groups=1, taps=2, mlp=moe(experts=4, top=4, ff=8, shared=8))],
                  **kw)


def to_bfloat16_values(values):
    """The nearest values that bfloat16 holds (ties to even), still as float32."""
    bits = np.ascontiguousarray(values, dtype=np.float32).view(np.uint32).astype(np.uint64)
    bits = (bits + 0x7FFF + ((bits >> 16) & 1)) & 0xFFFF0000
    return bits.astype(np.uint32).view(np.float32).reshape(np.shape(values))


def make_model(folder, raw, seed=0, bend=None, matrix_scale=1.0, bfloat16_values=False):
    """Write config.json and model.safetensors (32-bit) with random weights: matrices N(0, 0.05)
    times ``matrix_scale``, gains U(0.5, 1.5), norm offsets N(0, 0.1), biases N(0, 0.02).
    ``bend(tensors)`` may change them before they are written.  ``bfloat16_values``: every value is
    one that bfloat16 holds, as in a model that was stored in that type, so that a bfloat16
    engine and the plain model compute with the same weights."""
    parsed = config_from_dict(raw)
    tensors = random_tensors(describe_model(parsed), seed, "varied")
    for name, values in tensors.items():
        if values.ndim == 2 and not name.endswith("conv") and name != "embed":
            values *= matrix_scale
        if name.endswith("conv"):
            values *= 8.0                   # taps of about 0.4: every tap matters
    if bend is not None:
        bend(tensors)
    if bfloat16_values:
        tensors = {name: to_bfloat16_values(values) for name, values in tensors.items()}
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as handle:
        json.dump(raw, handle)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors, {name: "F32" for name in tensors})
    return folder


def sharpen(factor):
    """Scale the attention's query projections so that scores spread out and single keys matter
    (with small random weights attention is nearly uniform and a lost key would not show)."""
    def bend(tensors):
        for name, values in tensors.items():
            if name.endswith(".left.q"):
                values *= factor
    return bend


_cache = {}


def plain_logits(folder, tokens, streams=None):
    key = (folder, tuple(tokens))
    if key not in _cache or streams is not None:
        model_config, tensors = plain.load_model(folder)
        _cache[key] = plain.forward(model_config, tensors, list(tokens), streams)
    return _cache[key]
