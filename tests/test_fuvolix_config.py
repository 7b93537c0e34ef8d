"""Fuvolix without a device: its configuration reader, its description, the caches it asks
for, and the plain implementation's own consistency."""

import copy

import numpy as np
import pytest

import fuvolix_helpers as fx
import plain_fuvolix as plain
from mini_llm_b200.cache.manager import CacheManager
from mini_llm_b200.config import ConfigError, config_from_dict, describe_model
from mini_llm_b200.engine.model import Model
from mini_llm_b200.parts import FixedState, PagedKV
from mini_llm_b200.weights.loader import collect_specs


def test_configuration_round_trip_and_description():
    raw = fx.full_stack()
    parsed = config_from_dict(raw)
    assert parsed.architecture == "Fuvolix" and parsed.to_dict() == raw
    spec = describe_model(parsed)
    assert spec.keeps_layer_results and spec.embedding_norm.kind == "grouped_rms_norm" and spec.max_positions is None
    kinds = [layer.parts["mixer"].kind for layer in spec.layers]
    assert kinds == ["latent_attention", "gated_matrix_memory", "decaying_matrix_memory", "latent_attention",
                     "gated_matrix_memory"]
    assert ["feed_forward" in layer.parts for layer in spec.layers] == [True, False, True, False, True]
    names = collect_specs(Model(spec).parts())
    assert names["l2.dwa"].shape == (4,) and names["l0.canon1"].shape == (96, 3) and names["embed"].shape == (211, 96)
    assert names["l0.mix.dkv"].shape == (48, 96) and names["l3.mix.q"].shape == (2 * 24, 96)
    assert "l1.mlp.up" not in names and names["l2.mlp.up"].shape == (72, 96)


@pytest.mark.parametrize("change, key", [
    (lambda c: c.pop("vocab"), "vocab"),
    (lambda c: c["norm"].pop("groups"), "norm.groups"),
    (lambda c: c["norm"].update(groups=5), "norm.groups"),
    (lambda c: c["canon"].update(taps=0), "canon.taps"),
    (lambda c: c["layers"][0].update(type="window_attention"), "layers[0].type"),
    (lambda c: c["layers"][0]["mixer"].pop("kv_rank"), "layers[0].mixer.kv_rank"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "layers[0].mixer.rot.dims"),
    (lambda c: c["layers"][1]["mixer"].update(gate_cap="high"), "layers[1].mixer.gate_cap"),
    (lambda c: c["layers"][2]["mixer"].update(decay=[0.5]), "layers[2].mixer.decay"),
    (lambda c: c["layers"][2]["mlp"].update(kind="routed"), "layers[2].mlp.kind"),
    (lambda c: c.update(layers=[]), "layers"),
])
def test_configuration_errors_name_the_key(change, key):
    raw = copy.deepcopy(fx.full_stack())
    change(raw)
    with pytest.raises(ConfigError) as error:
        config_from_dict(raw)
    assert f"'{key}'" in str(error.value)


def test_a_layer_with_two_caches_gets_one_per_part():
    spec = describe_model(config_from_dict(fx.full_stack()))
    needs = Model(spec).cache_needs()
    assert needs[0] == {"mixer": PagedKV(1, 48, None, has_values=False), "input_filter": FixedState((2, 96), "float32")}
    manager = CacheManager(needs, 8, 10, 2, 80)
    by_need = {group.need: group.entries for group in manager.groups}
    assert by_need[FixedState((2, 96), "float32")] == [(i, "input_filter") for i in range(5)]
    assert by_need[PagedKV(1, 48, None, has_values=False)] == [(0, "mixer")]
    assert manager.entry_group[(3, "mixer")][0] != manager.entry_group[(0, "mixer")][0]     # other row width, other pool
    slot = manager.open()
    assert manager.reserve(slot, 20) and manager.pages_held(slot).count(3) == 2
    manager.commit(slot, 20)
    manager.close(slot)
    manager.check()
    # without taps there is no filter state, and the layer's cache is the mixer's alone
    bare = Model(describe_model(config_from_dict(fx.config([fx.lightning()], taps=1)))).cache_needs()
    assert bare == [{"mixer": FixedState((5 * 8 * 16,), "float32")}]


def test_plain_mixers_do_not_look_ahead():
    """The plain implementation's own check: logits at position p depend on tokens 0..p only."""
    raw = fx.full_stack()
    parsed = config_from_dict(raw)
    from mini_llm_b200.weights.random_init import random_tensors
    tensors = {k: v.astype(np.float64) for k, v in random_tensors(describe_model(parsed), 1, "varied").items()}
    tokens = [int(t) for t in np.random.default_rng(1).integers(0, 211, 20)]
    whole = plain.forward(raw, tensors, tokens)
    part = plain.forward(raw, tensors, tokens[:13])
    np.testing.assert_allclose(whole[:13], part, atol=1e-12)
    changed = list(tokens)
    changed[15] = (changed[15] + 1) % 211
    np.testing.assert_allclose(plain.forward(raw, tensors, changed)[:15], whole[:15], atol=1e-12)
