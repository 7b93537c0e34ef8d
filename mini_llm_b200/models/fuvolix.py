"""Fuvolix as a model description.

A decoder-only stack.  The embedded tokens are normed; every layer norms its sublayers on both
sides (the arrangement "sandwich_norm"), reads its mixer's input through a short causal
convolution, and hands on a learned weighted sum of the embedding output and all layer results
so far; the head is the token table itself behind a final norm.  All norms divide groups of the
width by their root mean square.  Each layer names its mixer: attention over a shared latent
(``latent_attention``), the gated matrix memory of xLSTM (``mlstm``), or lightning attention, a
matrix memory with a fixed decay per head (``lightning``); a layer may have a feed-forward with
the square of relu or none.

Tensor names: ``embed``, ``embed.norm``, ``final.norm``; layer i: ``l<i>.norm1``, ``.norm1b``,
``.norm2``, ``.norm2b``, ``.canon1`` [width, taps], ``.dwa`` [i + 2], ``.mix.*`` and ``.mlp.up`` /
``.mlp.down``; matrices are stored [out, in].
"""

from __future__ import annotations

from ..config.fuvolix import FuvolixConfig
from ..config.registry import register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, RunEntry


def _mixer(kind: str, sizes: dict, prefix: str, width: int, eps: float) -> PartSpec:
    if kind == "latent_attention":
        return PartSpec("latent_attention", prefix, {
            "width": width, "n_heads": sizes["heads"], "head_size": sizes["dim"], "rotated_size": sizes["rot_dim"],
            "value_size": sizes["vdim"], "latent_size": sizes["kv_rank"], "score_scale": sizes["scale"],
            "rotary_base": sizes["rot"]["base"], "rotary_dims": sizes["rot"]["dims"], "eps": eps})
    common = {"width": width, "n_heads": sizes["heads"], "key_size": sizes["dim"], "value_size": sizes["vdim"], "eps": eps}
    if kind == "mlstm":
        return PartSpec("gated_matrix_memory", prefix, {**common, "gate_cap": sizes["gate_cap"]})
    if kind == "lightning":
        return PartSpec("decaying_matrix_memory", prefix, {**common, "decay": tuple(sizes["decay"])})
    raise ValueError(f"unknown mixer '{kind}'")


def describe(config: FuvolixConfig) -> ModelSpec:
    width, eps = config.width, config.norm_eps

    def norm(prefix, name):
        return PartSpec("grouped_rms_norm", prefix, {"width": width, "eps": eps, "groups": config.norm_groups, "name": name})

    layers = []
    for index, layer in enumerate(config.layers):
        prefix = f"l{index}"
        parts = {
            "norm_1": norm(prefix, "norm1"),
            "input_filter": PartSpec("causal_taps", prefix, {"width": width, "taps": config.canon_taps, "name": "canon1"}),
            "mixer": _mixer(layer["type"], layer["mixer"], f"{prefix}.mix", width, eps),
            "norm_1b": norm(prefix, "norm1b"),
            "depth_mix": PartSpec("depth_weighted_sum", prefix, {"n_inputs": index + 2, "name": "dwa"}),
        }
        if layer["mlp"] is not None:
            parts.update({
                "norm_2": norm(prefix, "norm2"),
                "feed_forward": PartSpec("dense_mlp", f"{prefix}.mlp", {
                    "width": width, "inner": layer["mlp"]["ff"], "activation": "relu_squared", "up_name": "up",
                    "down_name": "down", "stored_in_out": False, "bias": False, "weight_suffix": ""}),
                "norm_2b": norm(prefix, "norm2b"),
            })
        layers.append(LayerSpec("sandwich_norm", parts))
    return ModelSpec(
        hidden_size=width,
        vocab_size=config.vocab,
        max_positions=None,
        embedding=PartSpec("token_embedding", "", {"vocab_size": config.vocab, "width": width, "name": "embed"}),
        position=None,
        embedding_norm=norm("embed", "norm"),
        keeps_layer_results=True,
        layers=tuple(layers),
        order=tuple(RunEntry(i) for i in range(len(layers))),
        final_norm=norm("final", "norm"),
        head=PartSpec("linear_head", "", {"vocab_size": config.vocab, "width": width, "weight_name": "embed"}),
    )


register_architecture("Fuvolix", FuvolixConfig, describe)
