"""Configuration, tensor list, order of layers, and the plain mechanisms of the Sofunex decoder (no GPU)."""
import copy

import numpy as np
import pytest

from sofunex_cases import CASES, random_config, stored, tensor_shapes


def _spec(raw):
    from xeno_rt_b200.config import config_from_dict
    arch, config = config_from_dict(raw)
    return arch, config, arch.build_spec(config)


@pytest.mark.parametrize("name", list(CASES))
def test_the_spec_expects_exactly_the_tensors_of_the_design(name):
    raw = CASES[name][0]
    arch, config, spec = _spec(raw)
    assert arch.name == "Sofunex"
    spec.validate()
    got = {e.name: tuple(e.shape) for e in spec.expected_tensors()}
    assert got == {k: tuple(v) for k, v in tensor_shapes(raw).items()}
    assert config.to_dict() == raw and _spec(config.to_dict())[1] == config


def test_random_configurations_give_their_tensors_too():
    for seed in range(40):
        raw = copy.deepcopy(random_config(np.random.default_rng(seed)))
        spec = _spec(raw)[2]
        assert {e.name: tuple(e.shape) for e in spec.expected_tensors()} == {k: tuple(v) for k, v in tensor_shapes(raw).items()}


def test_the_rank_of_the_decay_product_comes_from_the_tensors_shapes():
    from xeno_rt_b200.config import config_from_dict
    from xeno_rt_b200.core import ConfigError
    raw = CASES["mixed"][0]
    arch, config = config_from_dict(stored(raw))
    with pytest.raises(ConfigError) as err:
        arch.build_spec(config)
    assert "decay_rank" in str(err.value)
    full = config.with_tensor_shapes(tensor_shapes(raw))
    assert [l["mixer"]["right"]["decay_rank"] for l in full.layers] == [8, 12, 8, 16]
    assert {e.name for e in arch.build_spec(full).expected_tensors()} == set(tensor_shapes(raw))


def test_a_loop_repeats_its_layers_with_a_cache_each_and_begins_every_pass_with_its_row():
    raw = CASES["mixed"][0]
    spec = _spec(raw)[2]
    assert [p.layer for p in spec.schedule] == [0, 1, 2, 1, 2, 1, 2, 3]
    assert [p.before for p in spec.schedule] == [None, "loop_step_0", None, "loop_step_1", None, "loop_step_2", None, None]
    assert all(p.cache_from is None for p in spec.schedule)
    assert sorted((name, part.params["row"]) for name, part in spec.stream_parts.items()) == \
        [("loop_step_0", 0), ("loop_step_1", 1), ("loop_step_2", 2)]
    wide = _spec(CASES["wide"][0])[2]   # a loop that begins with the first layer
    assert [(p.layer, p.before) for p in wide.schedule] == [(0, "loop_step_0"), (1, None), (0, "loop_step_1"), (1, None), (2, None)]
    assert [p.before for p in _spec(CASES["odd"][0])[2].schedule] == [None, None, None] and not _spec(CASES["odd"][0])[2].stream_parts
    once = copy.deepcopy(raw)
    once["loop"]["times"] = 1           # one pass still begins with its row
    assert [p.before for p in _spec(once)[2].schedule] == [None, "loop_step_0", None, None]


def test_what_is_not_there_means_none():
    """No key, null and (for the taps) 0 say the same: no convolution, rotation, scaling, window, groups, shared
    expert, feed-forward or loop; factors that are not given are 1."""
    raw = copy.deepcopy(CASES["mixed"][0])
    left = raw["layers"][0]["mixer"]["left"]
    left.update({"conv": 0, "rot": None, "mask": None})
    raw["layers"][3]["mixer"]["left"]["rot"]["scaling"] = None
    raw["layers"][1]["mlp"].update({"shared": None})
    raw["layers"][1]["mlp"]["router"]["groups"] = None
    raw["layers"][0]["mlp"] = None
    raw["loop"] = None
    for key in ("left_scale", "right_scale"):
        raw["layers"][2]["mixer"].pop(key)
    raw.pop("embedding")
    raw.pop("residual_mult")
    spec = _spec(raw)[2]
    attention = spec.layers[0].parts["mixer"][1].params["branches"][0]["params"]
    assert attention["conv"] is None and attention["window"] is None and attention["position"]["kind"] == "none"
    assert spec.layers[3].parts["mixer"][1].params["branches"][0]["params"]["position"]["params"]["divide"] == 1.0
    experts = spec.layers[1].parts["ffn"][1].params
    assert "shared" not in experts and (experts["groups"], experts["keep_groups"]) == (1, 1)
    assert "ffn" not in spec.layers[0].parts and not spec.stream_parts and len(spec.schedule) == 4
    assert [b["scale"] for b in spec.layers[2].parts["mixer"][1].params["branches"]] == [1.0, 1.0]
    assert "gain" not in spec.layers[0].parts["mixer_post"][1].params or spec.layers[0].parts["mixer_post"][1].params["gain"] == 1.0
    assert spec.embedding.params["scale"] == 1.0
    names = {e.name for e in spec.expected_tensors()}
    assert "l0.mix.left.q.conv" not in names and "loop.step" not in names and "l1.mlp.shared.up" not in names


def test_what_a_layer_is_made_of():
    spec = _spec(CASES["mixed"][0])[2]
    first, third = spec.layers[0], spec.layers[2]
    assert list(first.parts) == ["mixer_norm", "mixer_shift", "mixer", "mixer_post", "ffn_norm", "ffn", "ffn_post"]
    assert list(third.parts) == ["mixer_norm", "mixer_shift", "mixer", "mixer_post"]
    assert first.parts["mixer_post"][1].params["gain"] == 0.8 and "gain" not in first.parts["mixer_norm"][1].params
    mixer = first.parts["mixer"][1]
    assert mixer.params["combine"] == "weighted" and [b["scale"] for b in mixer.params["branches"]] == [0.7, 1.1]
    l = mixer.params["branches"][0]["params"]
    assert (l["conv"], l["window"], l["v_norm"], l["qk_norm"], l["bias"], l["o_bias"]) == (3, 40, "unit", "whole", True, True)
    assert l["position"]["params"]["divide"] == 4.0 and l["position"]["params"]["pairing"] == "split_half"
    experts = spec.layers[1].parts["ffn"][1].params
    assert (experts["scores"], experts["group_best"], experts["normalize"], experts["weight_scale"], experts["shared"]) == \
        ("sigmoid", 2, True, 1.5, 40)
    assert "shared" not in spec.layers[3].parts["ffn"][1].params and spec.layers[3].parts["ffn"][1].params["groups"] == 1
    assert spec.embedding.params["scale"] == 3.5


def test_every_bad_key_is_reported_in_one_error():
    from xeno_rt_b200.core import ConfigError
    raw = copy.deepcopy(CASES["mixed"][0])
    raw["width"] = 0
    raw["layers"][0]["mixer"]["left"]["kv_heads"] = 3           # 4 heads are no multiple
    raw["layers"][0]["mixer"]["left"]["mask"].pop("size")
    raw["layers"][0]["mixer"]["left"]["rot"]["dims"] = 18       # beyond the head
    raw["layers"][0]["mixer"]["left"]["conv"] = -2
    raw["layers"][1]["mlp"]["router"]["groups"]["count"] = 3    # 8 experts are no multiple
    raw["layers"][1]["mixer"].pop("right")
    raw["layers"][2]["mlp"] = {"kind": "swiglu"}
    raw["layers"][3]["mlp"]["router"]["top"] = 7                # of 6 experts
    raw["layers"].append({"type": "gla", "mixer": {}, "mlp": None})
    raw["loop"]["stop"] = 9
    raw["norm"] = {}
    raw["residual_mult"] = 0
    with pytest.raises(ConfigError) as err:
        _spec(raw)
    text = str(err.value)
    for piece in ("config.width", "kv_heads", "mask.size", "rot.dims", ".conv", "equal groups", "right is missing",
                  "kind 'swiglu'", "top 7", "'gla'", "loop", "norm.eps", "residual_mult"):
        assert piece in text, piece


# ----------------------------------------------------------------------------- the plain mechanisms themselves
def test_plain_token_shift_and_convolution_read_only_the_past():
    from plain import sofunex
    rng = np.random.default_rng(0)
    h, shift = rng.normal(size=(6, 5)), rng.uniform(size=5)
    out = sofunex.token_shift(h, shift)
    assert np.allclose(out[0], h[0] * (1 - shift)) and np.allclose(out[3], h[3] + (h[2] - h[3]) * shift)
    u, w = rng.normal(size=(7, 3)), rng.normal(size=(3, 4))
    y = sofunex.short_convolution(u, w)
    assert np.allclose(y[0], w[:, 3] * u[0]) and np.allclose(y[5], sum(w[:, j] * u[2 + j] for j in range(4)))
    later = u.copy()
    later[4:] += 1.0
    assert np.allclose(sofunex.short_convolution(later, w)[:4], y[:4])


def test_plain_delta_step_removes_along_the_unit_key_from_the_old_state():
    from plain import sofunex
    rng = np.random.default_rng(1)
    d = 6
    S, r, k, v = rng.normal(size=(d, d)), rng.normal(size=d), rng.normal(size=d), rng.normal(size=d)
    ones, none = np.ones(d), np.zeros(d)
    # no decay, full removal, nothing written: what the state answered along the key is gone
    n = k / np.sqrt(k @ k + 1e-6)
    after, _ = sofunex.delta_step(S, r, np.zeros(d), np.zeros(d), ones, ones)
    assert np.allclose(after, S)                      # a zero key removes nothing
    after, out = sofunex.delta_step(S, r, k, none, ones, ones)
    assert np.allclose(n @ after, (n @ S) * (1 - n @ n), atol=1e-5) and np.allclose(out, after.T @ r)
    # both corrections read the state as it came: decay 0.5 and removal together
    after, _ = sofunex.delta_step(S, r, k, v, 0.5 * ones, 0.25 * ones)
    assert np.allclose(after, 0.5 * S - np.outer(0.25 * n, n @ S) + np.outer(k, v))


def test_plain_routing_counts_groups_by_two_and_weighs_without_the_correction():
    from plain import sofunex
    d = 4
    w = {"m.router": np.zeros((6, d)), "m.correction": np.array([0.4, -0.9, 0.1, 0.1, 0.3, -2.0])}
    w["m.router"][:, 0] = [0.0, 2.0, 1.0, 1.0, -1.0, 3.0]
    mlp = {"router": {"experts": 6, "top": 2, "scale": 3.0, "groups": {"count": 3, "keep": 1}}}
    h = np.array([1.0, 0, 0, 0])
    s = 1 / (1 + np.exp(-w["m.router"][:, 0]))
    choice = s + w["m.correction"]
    worth = [choice[0] + choice[1], choice[2] + choice[3], choice[4] + choice[5]]
    assert int(np.argmax(worth)) == 1                                   # the pair of middling experts beats the best single one
    chosen, weights, margin = sofunex.route(h, w, "m.", mlp)
    assert chosen == [2, 3] and np.allclose(weights, 3.0 * s[[2, 3]] / s[[2, 3]].sum()) and np.isclose(weights.sum(), 3.0)
    assert np.isclose(margin, worth[1] - sorted(worth)[-2])
    mlp["router"]["groups"] = {"count": 3, "keep": 3}
    chosen, weights, _ = sofunex.route(h, w, "m.", mlp)
    assert chosen == [0, 2]                                             # by choice score (a tie goes to the lower number); expert 5 has the best plain score
    w["m.correction"] = np.full(6, -5.0)                                # choice scores below zero: an expert of a group
    mlp["router"]["groups"] = {"count": 3, "keep": 1}                   # that is not kept counts as minus infinity, not as 0
    assert sofunex.route(h, w, "m.", mlp)[0] == [2, 3]
