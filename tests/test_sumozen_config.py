"""Sumozen without a device: the configuration's round trip and its errors, what the layers keep
per request, and the plain model's own causality."""

import copy

import numpy as np
import pytest

import sumozen_helpers as sz
from mini_llm_b200.config import ConfigError, config_from_dict, describe_model
from mini_llm_b200.engine.model import Model
from mini_llm_b200.parts.spec import FixedState, PagedKV


def test_round_trip():
    raw = sz.full_stack()
    parsed = config_from_dict(raw)
    assert parsed.architecture == "Sumozen"
    assert parsed.to_dict() == raw
    assert config_from_dict(parsed.to_dict()) == parsed


def _without(raw, path):
    raw = copy.deepcopy(raw)
    node = raw
    for key in path[:-1]:
        node = node[key]
    del node[path[-1]]
    return raw


def _with(raw, path, value):
    raw = copy.deepcopy(raw)
    node = raw
    for key in path[:-1]:
        node = node[key]
    node[path[-1]] = value
    return raw


@pytest.mark.parametrize("change, named", [
    (lambda r: _without(r, ["vocab"]), "vocab"),
    (lambda r: _without(r, ["norm", "eps"]), "norm.eps"),
    (lambda r: _with(r, ["layers", 0, "type"], "hyena"), "layers[0].type"),
    (lambda r: _without(r, ["layers", 0, "mixer", "left", "kv_heads"]), "layers[0].mixer.left.kv_heads"),
    (lambda r: _with(r, ["layers", 0, "mixer", "left", "heads"], 3), "layers[0].mixer.left.heads"),
    (lambda r: _with(r, ["layers", 0, "mixer", "left", "rot", "dims"], 13), "layers[0].mixer.left.rot.dims"),
    (lambda r: _without(r, ["layers", 0, "mixer", "left", "rot", "scaling", "slow"]), "layers[0].mixer.left.rot.scaling.slow"),
    (lambda r: _with(r, ["layers", 0, "mixer", "right", "dim"], "wide"), "layers[0].mixer.right.dim"),
    (lambda r: _without(r, ["layers", 0, "mixer", "right_scale"]), "layers[0].mixer.right_scale"),
    (lambda r: _with(r, ["layers", 1, "mixer", "norm_groups"], 5), "layers[1].mixer.norm_groups"),
    (lambda r: _with(r, ["layers", 1, "mixer", "groups"], 3), "layers[1].mixer.heads"),
    (lambda r: _with(r, ["layers", 0, "mlp", "router", "top"], 9), "layers[0].mlp.router.top"),
    (lambda r: _with(r, ["layers", 0, "mlp", "kind"], "dense"), "layers[0].mlp.kind"),
    (lambda r: _without(r, ["layers", 0, "mlp", "expert"]), "layers[0].mlp.expert"),
])
def test_errors_name_their_key(change, named):
    with pytest.raises(ConfigError) as error:
        config_from_dict(change(sz.full_stack()))
    assert f"'{named}" in str(error.value)


def test_what_the_layers_keep():
    model = Model(describe_model(config_from_dict(sz.full_stack())))
    needs = model.cache_needs()
    first = needs[0]
    assert set(first) == {"mixer.left.kv", "mixer.left.taps", "mixer.right.state", "mixer.right.taps"}
    assert first["mixer.left.kv"] == PagedKV(2, 16, None, value_size=24)
    assert first["mixer.left.taps"] == FixedState((2, 4 * 16 + 2 * 16 + 2 * 24), "float32")
    assert first["mixer.right.state"] == FixedState((4 * 12 * 20,), "float32")
    assert first["mixer.right.taps"] == FixedState((3, 2 * 2 * 12 + 4 * 20), "float32")
    assert needs[1] == {"mixer.state": FixedState((4 * 20 * 12,), "float32"), "mixer.taps": FixedState((3, 4 * 12 + 2 * 2 * 20), "float32")}
    assert model.graph_safe
    # one tap: nothing to keep for the convolution
    lone = Model(describe_model(config_from_dict(sz.config([sz.mamba(taps=1)]))))
    assert lone.cache_needs()[0] == {"mixer.state": FixedState((4 * 20 * 12,), "float32")}


def test_yarn_frequencies_against_the_formula():
    from mini_llm_b200.parts.rotary import rotary_frequencies
    import plain_sumozen as plain
    for rot in ({"base": 300.0, "dims": 12, "scaling": sz.YARN}, {"base": 10000.0, "dims": 64, "scaling": None},
                {"base": 5e5, "dims": 32, "scaling": {"factor": 16.0, "original": 128, "fast": 32.0, "slow": 1.0}}):
        got, amplitude = rotary_frequencies(rot["base"], rot["dims"], rot["scaling"])
        want, want_amplitude = plain.yarn_frequencies(rot)
        np.testing.assert_allclose(got, want, rtol=1e-14)
        assert abs(amplitude - want_amplitude) < 1e-15


def test_the_plain_model_is_causal(tmp_path):
    import plain_sumozen as plain
    folder = sz.make_model(str(tmp_path / "m"), sz.full_stack(), seed=1, matrix_scale=2.0)
    config, tensors = plain.load_model(folder)
    tokens = np.random.default_rng(0).integers(0, 211, 20).tolist()
    full = plain.forward(config, tensors, tokens)
    short = plain.forward(config, tensors, tokens[:11])
    np.testing.assert_allclose(full[:11], short, atol=1e-10)
    changed = list(tokens)
    changed[15] = (changed[15] + 1) % 211
    np.testing.assert_allclose(plain.forward(config, tensors, changed)[:15], full[:15], atol=1e-10)
    assert np.abs(plain.forward(config, tensors, changed)[15:] - full[15:]).max() > 1e-6
