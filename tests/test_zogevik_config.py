"""Configuration, tensor list and the plain routing, softmax and rotations of the Zogevik decoder (no GPU)."""
import copy

import numpy as np
import pytest

from zogevik_cases import CASES, random_config, tensor_shapes


def _spec(raw):
    from xeno_rt_b200.config import config_from_dict
    arch, config = config_from_dict(raw)
    return arch, config, arch.build_spec(config)


@pytest.mark.parametrize("name", list(CASES))
def test_the_spec_expects_exactly_the_tensors_of_the_design(name):
    raw = CASES[name][0]
    arch, config, spec = _spec(raw)
    assert arch.name == "Zogevik"
    spec.validate()
    got = {e.name: tuple(e.shape) for e in spec.expected_tensors()}
    assert got == {k: tuple(v) for k, v in tensor_shapes(raw).items()}
    assert config.to_dict() == raw and _spec(config.to_dict())[1] == config


def test_random_configurations_give_their_tensors_too():
    for seed in range(40):
        raw = copy.deepcopy(random_config(np.random.default_rng(seed)))
        for layer in raw["layers"]:
            layer["mixer"]["scale"] = float(layer["mixer"]["scale"])
        spec = _spec(raw)[2]
        assert {e.name: tuple(e.shape) for e in spec.expected_tensors()} == {k: tuple(v) for k, v in tensor_shapes(raw).items()}


def test_a_layer_that_reads_another_layers_keys_is_scheduled_on_its_cache():
    raw = CASES["odd"][0]
    spec = _spec(raw)[2]
    assert [p.cache_from for p in spec.schedule] == [None, None, 1, None, 1]
    names = {e.name for e in spec.expected_tensors()}
    assert "l1.mix.k" in names and "l2.mix.k" not in names and "l4.mix.k.norm" not in names and "l4.mix.v" not in names
    assert "l1.norm2" not in names and "l2.norm2" in names   # a layer without a feed-forward has no second norm


def test_every_bad_key_is_reported_in_one_error():
    from xeno_rt_b200.core import ConfigError
    raw = copy.deepcopy(CASES["mixed"][0])
    raw["width"] = 0
    raw["layers"][0]["mixer"]["kv_heads"] = 3           # 4 heads are no multiple
    raw["layers"][0]["mixer"]["mask"].pop("size")
    raw["layers"][0]["mixer"]["rot"]["dims"] = 18       # beyond the head
    raw["layers"][0]["mlp"]["router"]["groups"]["count"] = 3   # 8 experts are no multiple
    raw["layers"][1]["mixer"]["rot"]["dims"] = 4        # a latent layer rotates all of rot_dim
    raw["layers"][1]["mlp"] = {"kind": "swiglu"}
    raw["layers"][2]["mixer"]["kv_from"] = 1            # a latent layer has no keys to give
    raw["layers"][3]["mlp"]["router"]["top"] = 5        # two groups of 2 are kept
    raw["layers"].append({"type": "conv", "mixer": {}, "mlp": None})
    raw["norm"] = {}
    with pytest.raises(ConfigError) as err:
        _spec(raw)
    text = str(err.value)
    for piece in ("width", "kv_heads", "mask", "rot.dims 18", "3 equal groups", "rot.dims 4", "swiglu", "kv_from", "top 5",
                  "'conv'", "eps"):
        assert piece in text, piece


def test_a_reader_must_match_its_owner_and_come_after_it():
    from xeno_rt_b200.core import ConfigError
    for key, value in (("dim", 32), ("kv_heads", 1), ("vdim", 8)):
        raw = copy.deepcopy(CASES["mixed"][0])
        raw["layers"][2]["mixer"][key] = value
        with pytest.raises(ConfigError):
            _spec(raw)
    raw = copy.deepcopy(CASES["mixed"][0])
    raw["layers"][2]["mixer"]["rot"]["base"] = 5.0
    with pytest.raises(ConfigError):
        _spec(raw)
    raw = copy.deepcopy(CASES["mixed"][0])
    raw["layers"][0]["mixer"]["kv_from"] = 2
    with pytest.raises(ConfigError):
        _spec(raw)
    raw = copy.deepcopy(CASES["odd"][0])
    raw["layers"][4]["mixer"]["kv_from"] = 2            # layer 2 reads layer 1 itself
    with pytest.raises(ConfigError):
        _spec(raw)


def test_the_plain_routing_keeps_the_best_groups_and_the_scores_as_they_are():
    from plain import zogevik
    scores = np.array([0.05, 0.30, 0.02, 0.03, 0.25, 0.20, 0.10, 0.05])
    # groups of two: bests 0.30, 0.03, 0.25, 0.10; two kept: 0 and 2; of experts 0, 1, 4, 5 the best three
    assert zogevik.choose(scores, 3, 4, 2) == [1, 4, 5]
    assert zogevik.choose(scores, 2, 4, 1) == [1, 0]     # expert 5's 0.20 is larger but its group is not kept
    assert zogevik.choose(scores, 3, 1, 1) == [1, 4, 5]
    assert zogevik.choose(np.array([0.25, 0.25, 0.25, 0.25]), 2, 2, 1) == [0, 1]   # the lower number wins a tie
    h = np.array([[1.0, -2.0, 0.5]])
    w = {"router": np.array([[1.0, 0, 0], [0, 1.0, 0], [0, 0, 1.0], [1.0, 1.0, 1.0]])}
    for e in range(4):
        w[f"e{e}.up"] = np.eye(3) * (e + 1)
        w[f"e{e}.down"] = np.eye(3)
    s = zogevik.router_scores(h, w["router"])[0]
    assert abs(s.sum() - 1) < 1e-12
    out = zogevik.moe_ff(h, w, {"router": {"experts": 4, "top": 2, "groups": {"count": 2, "keep": 1}}})
    want = s[0] * zogevik.gelu_erf(h[0]) + s[1] * zogevik.gelu_erf(2 * h[0])   # group 0 holds the best score
    assert np.allclose(out[0], want) and s[0] + s[1] < 0.9                      # not renormalized


def test_the_plain_softmax_with_a_sink_gives_less_than_an_average():
    from plain import zogevik
    p = zogevik.softmax_weights([-30.0, -31.0], sink=True)
    assert p.sum() < 1e-12
    p = zogevik.softmax_weights([0.0, 0.0, 0.0], sink=True)
    assert np.allclose(p, 0.25)
    p = zogevik.softmax_weights([800.0, 799.0], sink=True)
    assert abs(p.sum() - 1) < 1e-12
    assert abs(zogevik.softmax_weights([0.0, 0.0, 0.0], sink=False).sum() - 1) < 1e-12


def test_the_plain_rotations_pair_as_the_design_says():
    from plain import zogevik
    v = np.arange(1.0, 9.0)
    a = zogevik.angles(3, 4, 100.0)
    assert np.allclose(a, [3.0, 0.3])
    s = zogevik.rotate_split_half(v, 3, 4, 100.0)
    assert np.allclose(s[4:], v[4:]) and np.allclose(s[0], 1 * np.cos(3.0) - 3 * np.sin(3.0))
    assert np.allclose(s[3], 4 * np.cos(0.3) + 2 * np.sin(0.3))
    t = zogevik.rotate_interleaved(v, 3, 4, 100.0)
    assert np.allclose(t[4:], v[4:]) and np.allclose(t[0], 1 * np.cos(3.0) - 2 * np.sin(3.0))
    assert np.allclose(t[3], 4 * np.cos(0.3) + 3 * np.sin(0.3))
    assert np.allclose(zogevik.rotate_interleaved(v, 0, 8, 7.0), v)
