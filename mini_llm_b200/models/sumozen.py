"""Sumozen as a model description.

A decoder-only pre-norm stack: ``x <- x + mixer(norm1(x))``, then, if the layer has one,
``x <- x + ff(norm2(x))``; all norms divide by the root mean square and multiply by ``1 + w``.
A layer of type "parallel" runs two mixers side by side on the same input and adds
``left_scale * left + right_scale * right``: on the left a softmax attention whose projected
queries, keys and values pass a short causal convolution before rotary positions (interleaved
pairs, YaRN-scaled frequencies), with a tanh cap on the scores; on the right a gated delta rule.
A layer of type "mamba2" has a state-space mixer.  The feed-forward is a mixture of experts with
sigmoid scores and an optional shared expert.  The head has a matrix of its own.

Tensor names: ``embed``, ``final.norm``, ``head``; layer i: ``l<i>.norm1``, ``l<i>.norm2``,
``l<i>.mix.*`` (``left.*`` / ``right.*`` in a parallel layer) and ``l<i>.mlp.*``; matrices are
stored [out, in].
"""

from __future__ import annotations

from ..config.registry import register_architecture
from ..config.sumozen import SumozenConfig
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, RunEntry


def _mixer(kind: str, sizes: dict, prefix: str, width: int, eps: float) -> PartSpec:
    if kind == "mamba2":
        return PartSpec("state_space_duality", prefix, {
            "width": width, "n_heads": sizes["heads"], "value_size": sizes["vdim"], "state_size": sizes["state"],
            "n_groups": sizes["groups"], "norm_groups": sizes["norm_groups"], "taps": sizes["conv"], "eps": eps})
    left, right = sizes["left"], sizes["right"]
    rotation = PartSpec("interleaved_rotary", f"{prefix}.left", {
        "base": left["rot"]["base"], "dims": left["rot"]["dims"],
        "scaling": tuple(sorted(left["rot"]["scaling"].items())) if left["rot"]["scaling"] else None})
    attention = PartSpec("filtered_attention", f"{prefix}.left", {
        "width": width, "n_heads": left["heads"], "n_kv_heads": left["kv_heads"], "key_size": left["dim"],
        "value_size": left["vdim"], "score_scale": left["scale"], "softcap": left["softcap"], "taps": left["conv"],
        "position": rotation})
    memory = PartSpec("gated_delta_memory", f"{prefix}.right", {
        "width": width, "n_heads": right["heads"], "n_qk_heads": right["kv_heads"], "key_size": right["dim"],
        "value_size": right["vdim"], "taps": right["conv"], "eps": eps})
    return PartSpec("parallel_mixers", prefix, {
        "branches": (("left", attention, sizes["left_scale"]), ("right", memory, sizes["right_scale"]))})


def describe(config: SumozenConfig) -> ModelSpec:
    width, eps = config.width, config.norm_eps

    def norm(prefix, name):
        return PartSpec("grouped_rms_norm", prefix, {"width": width, "eps": eps, "groups": 1, "name": name, "unit_offset": True})

    layers = []
    for index, layer in enumerate(config.layers):
        prefix = f"l{index}"
        parts = {"norm_1": norm(prefix, "norm1"), "mixer": _mixer(layer["type"], layer["mixer"], f"{prefix}.mix", width, eps)}
        mlp = layer["mlp"]
        if mlp is not None:
            parts["norm_2"] = norm(prefix, "norm2")
            parts["feed_forward"] = PartSpec("routed_experts", f"{prefix}.mlp", {
                "width": width, "n_experts": mlp["router"]["experts"], "top": mlp["router"]["top"],
                "expert_inner": mlp["expert"]["ff"], "shared_inner": mlp["shared"]["ff"] if mlp["shared"] else None})
        layers.append(LayerSpec("pre_norm", parts))
    return ModelSpec(
        hidden_size=width,
        vocab_size=config.vocab,
        max_positions=None,
        embedding=PartSpec("token_embedding", "", {"vocab_size": config.vocab, "width": width, "name": "embed"}),
        position=None,
        layers=tuple(layers),
        order=tuple(RunEntry(i) for i in range(len(layers))),
        final_norm=norm("final", "norm"),
        head=PartSpec("linear_head", "", {"vocab_size": config.vocab, "width": width, "weight_name": "head"}),
    )


register_architecture("Sumozen", SumozenConfig, describe)
