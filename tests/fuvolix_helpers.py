"""Shared by the Fuvolix tests: small configurations (none with the sizes of any released
model), model folders with random weights that a test may then bend, and the plain logits."""

import json
import os

import numpy as np

import plain_fuvolix as plain
from mini_llm_b200.config import config_from_dict, describe_model
from mini_llm_b200.weights.random_init import random_tensors
from mini_llm_b200.weights.safetensors_io import write_safetensors


def latent(heads=3, dim=16, rot_dim=8, vdim=24, kv_rank=40, scale=0.31, base=500.0, dims=None, ff=None):
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale,
                      "rot": {"base": base, "dims": rot_dim if dims is None else dims}},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def mlstm(heads=2, dim=24, vdim=40, gate_cap=9.0, ff=None):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": gate_cap},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def lightning(heads=5, dim=8, vdim=16, decay=None, ff=None):
    decay = decay if decay is not None else [0.5 + 0.499 * h / max(heads - 1, 1) for h in range(heads)]
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def config(layers, width=96, vocab=211, groups=3, taps=3, eps=1e-5):
    return {"architecture": "Fuvolix", "vocab": vocab, "width": width, "norm": {"eps": eps, "groups": groups},
            "canon": {"taps": taps}, "layers": list(layers)}


def full_stack(**kw):
    """All three mixers, with and without feed-forward, the attention twice."""
    return config([latent(ff=136), mlstm(), lightning(ff=72), latent(heads=2, dim=8, rot_dim=16, vdim=8, kv_rank=24, dims=12),
                   mlstm(heads=3, dim=8, vdim=8, gate_cap=4.0, ff=40)], **kw)


def make_model(folder, raw, seed=0, bend=None, matrix_scale=1.0):
    """Write config.json and model.safetensors (32-bit) with random weights: matrices N(0, 0.05)
    times ``matrix_scale``, gains U(0.5, 1.5), biases N(0, 0.02).  ``bend(tensors)`` may change
    them before they are written."""
    parsed = config_from_dict(raw)
    tensors = random_tensors(describe_model(parsed), seed, "varied")
    for name, values in tensors.items():
        if values.ndim == 2 and not name.endswith("canon1") and name != "embed":
            values *= matrix_scale
    if bend is not None:
        bend(tensors)
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as handle:
        json.dump(raw, handle)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors, {name: "F32" for name in tensors})
    return folder


def sharpen(factor):
    """Scale every query projection so that attention scores spread out and single keys matter
    (with small random weights attention is nearly uniform and a lost key would not show)."""
    def bend(tensors):
        for name, values in tensors.items():
            if name.endswith(".mix.q"):
                values *= factor
    return bend


_cache = {}


def plain_logits(folder, tokens, streams=None):
    key = (folder, tuple(tokens))
    if key not in _cache or streams is not None:
        model_config, tensors = plain.load_model(folder)
        _cache[key] = plain.forward(model_config, tensors, list(tokens), streams)
    return _cache[key]
