"""The Sazepel configuration, its model's tensor names, the cache it asks for, and the plain implementation's
mechanisms against each other (no GPU)."""
import copy

import numpy as np
import pytest
import torch

import plain_sazepel as plain
import sazepel_tiny as st
from alpacca_b200.config import ConfigError, config_from_dict
from alpacca_b200.config.sazepel import SazepelConfig
from alpacca_b200.engine.loading import build_model
from alpacca_b200.parts import KVSpec, StateSpec


@pytest.mark.parametrize("name", list(st.CONFIGS) + ["random3", "random8"])
def test_tensor_names_and_shapes(name):
    raw = st.CONFIGS[name] if name in st.CONFIGS else st.random_config(int(name[6:]))
    cfg = config_from_dict(raw)
    assert isinstance(cfg, SazepelConfig) and cfg.max_positions is None
    model = build_model(cfg, "float32", "cpu", 128)
    specs = {s.name: tuple(s.shape) for s in model.param_specs()}
    assert specs == st.tensor_shapes(raw)


@pytest.mark.parametrize("name", list(st.CONFIGS))
def test_cache_entries(name):
    """A retention keeps a float32 state per head; two mixers side by side keep one entry each, the attention's
    first: keys per key/value head, and a token's value heads side by side in one row."""
    raw = st.CONFIGS[name]
    model = build_model(config_from_dict(raw), "bfloat16", "cpu", 128)
    want = []
    for layer in raw["layers"]:
        mx = layer["mixer"]
        if layer["type"] == "parallel":
            lf = mx["left"]
            want.append(KVSpec(lf["kv_heads"], lf["dim"], None, value_heads=1, value_dim=lf["kv_heads"] * lf["vdim"]))
            mx = mx["right"]
        want.append(StateSpec((mx["heads"], mx["dim"], mx["vdim"]), torch.float32))
    assert model.cache_entry_specs() == want


def test_layers_with_the_same_rotation_share_one_table():
    raw = copy.deepcopy(st.TINY_R)
    raw["layers"].append(copy.deepcopy(raw["layers"][1]))
    model = build_model(config_from_dict(raw), "float32", "cpu", 128)
    a, b = model.spec.layers[1].mixer.position, model.spec.layers[3].mixer.position
    assert a is b and a is not model.spec.layers[0].mixer.right.position


def test_a_rotation_over_no_dims_is_none():
    model = build_model(config_from_dict(st.TINY_P), "float32", "cpu", 128)
    assert model.spec.layers[2].mixer.right.position is None
    assert model.spec.layers[0].mixer.right.position is not None


def _broken(change):
    raw = copy.deepcopy(st.TINY_P)
    change(raw)
    return raw


@pytest.mark.parametrize("change,words", [
    (lambda c: c["layers"][0].update(type="convolution"), "not supported"),
    (lambda c: c["layers"][1]["mixer"].update(decay=[0.5]), "decay"),
    (lambda c: c["layers"][1]["mixer"].update(decay=[0.5, 1.5]), "decay"),
    (lambda c: c["layers"][1]["mixer"].update(decay=[0.5, 0.0]), "decay"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=3), "cannot share"),
    (lambda c: c["layers"][0]["mixer"]["right"]["rot"].update(dims=3), "even"),
    (lambda c: c["layers"][0]["mixer"]["right"]["rot"].update(dims=10), "at most"),
    (lambda c: c["layers"][0]["mixer"]["right"]["rot"].pop("base"), "base"),
    (lambda c: c["layers"][0]["mixer"]["left"].pop("scale"), "scale"),
    (lambda c: c["layers"][0]["mixer"].pop("right"), "right"),
    (lambda c: c["layers"][1]["mixer"].pop("vdim"), "vdim"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "moe"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=5), "cannot be chosen"),
    (lambda c: c["layers"][0]["mlp"]["expert"].pop("ff"), "ff"),
    (lambda c: c["norm"].pop("eps"), "eps"),
    (lambda c: c.update(width=0), "width"),
    (lambda c: c.update(layers=[]), "layers"),
])
def test_every_fault_is_named(change, words):
    with pytest.raises(ConfigError) as err:
        config_from_dict(_broken(change))
    assert words in str(err.value)


def test_several_faults_in_one_error():
    raw = _broken(lambda c: (c["norm"].pop("eps"), c["layers"][1]["mixer"].update(decay=[2.0, 0.5]),
                             c["layers"][2]["mixer"]["left"].update(kv_heads=2)))
    with pytest.raises(ConfigError) as err:
        config_from_dict(raw)
    assert all(w in str(err.value) for w in ("eps", "decay", "cannot share"))


def test_the_configuration_goes_round():
    cfg = config_from_dict(st.TINY_Q)
    again = config_from_dict(cfg.to_dict())
    assert again.to_dict() == cfg.to_dict() and again.layers == st.TINY_Q["layers"]


# --- the plain implementation against itself: a mechanism written twice must agree ---

def test_plain_retention_is_a_decayed_sum():
    """o_t = sum over s <= t of decay^(t-s) (q_t . k_s) v_s, written as that sum, equals the recurrence; and the state
    that a prefix leaves carries the rest."""
    rng = np.random.default_rng(0)
    mx = {"heads": 2, "dim": 6, "vdim": 5, "decay": [0.8, 1.0], "rot": {"base": 50.0, "dims": 4}}
    E, T, eps = 9, 12, 1e-5
    w = {n: rng.normal(0, 0.4, s) for n, s in (("q", (12, E)), ("k", (12, E)), ("v", (10, E)), ("g", (10, E)), ("o", (E, 10)))}
    h = rng.normal(0, 1, (T, E))
    got, S = plain.retention(h, w, mx, eps)
    pos = np.arange(T)
    q = plain.turn_halves((h @ w["q"].T).reshape(T, 2, 6), pos, mx["rot"])
    k = plain.turn_halves((h @ w["k"].T).reshape(T, 2, 6), pos, mx["rot"]) / np.sqrt(6.0)
    v = (h @ w["v"].T).reshape(T, 2, 5)
    o = np.zeros((T, 2, 5))
    for t in range(T):
        for s in range(t + 1):
            for a in range(2):
                o[t, a] += mx["decay"][a] ** (t - s) * (q[t, a] @ k[s, a]) * v[s, a]
    want = (plain.unit(o, eps).reshape(T, 10) * plain.silu(h @ w["g"].T)) @ w["o"].T
    assert np.abs(got - want).max() < 1e-12
    first, S7 = plain.retention(h[:7], w, mx, eps)
    rest, S12 = plain.retention(h[7:], w, mx, eps, positions=np.arange(7, T), state=S7)
    assert np.abs(np.concatenate([first, rest]) - got).max() < 1e-12 and np.abs(S12 - S).max() < 1e-12


def test_plain_rotation_leaves_the_tail_and_keeps_lengths():
    rng = np.random.default_rng(1)
    x = rng.normal(0, 1, (5, 2, 10))
    y = plain.turn_halves(x, np.arange(5) + 3, {"base": 100.0, "dims": 6})
    assert np.array_equal(y[..., 6:], x[..., 6:])
    assert np.allclose((y[..., :6] ** 2).sum(-1), (x[..., :6] ** 2).sum(-1))
    # a pair is (i, i + 3): turning position 0 changes nothing, and the first pair turns by the position itself
    assert np.allclose(plain.turn_halves(x, np.zeros(5), {"base": 100.0, "dims": 6}), x)
    z = plain.turn_halves(np.eye(10)[None, None, 0], [2.0], {"base": 100.0, "dims": 6})[0, 0]
    assert np.allclose(z[[0, 3]], [np.cos(2.0), np.sin(2.0)]) and np.allclose(np.delete(z, [0, 3]), 0)


def test_plain_mixed_heads_with_the_identity_are_plain_attention():
    rng = np.random.default_rng(2)
    mx = {"heads": 4, "kv_heads": 2, "dim": 6, "vdim": 3, "scale": 0.7}
    E, T, eps = 8, 9, 1e-6
    w = {"q": rng.normal(0, 1, (24, E)), "k": rng.normal(0, 1, (12, E)), "v": rng.normal(0, 1, (6, E)),
         "g": rng.normal(0, 1, (12, E)), "o": rng.normal(0, 1, (E, 12)), "talk": np.eye(4)}
    h = rng.normal(0, 1, (T, E))
    got = plain.talking_attention(h, w, mx, eps)
    q = plain.unit((h @ w["q"].T).reshape(T, 4, 6), eps)
    k = plain.unit((h @ w["k"].T).reshape(T, 2, 6), eps)
    v = plain.unit((h @ w["v"].T).reshape(T, 2, 3), eps)
    o = np.zeros((T, 4, 3))
    for t in range(T):
        for a in range(4):
            s = np.array([q[t, a] @ k[j, a // 2] for j in range(t + 1)]) * 0.7
            p = np.exp(s - s.max())
            o[t, a] = (p / p.sum()) @ v[:t + 1, a // 2]
    want = (o.reshape(T, 12) * plain.sigmoid(h @ w["g"].T)) @ w["o"].T
    assert np.abs(got - want).max() < 1e-12
    # a mixing matrix that swaps heads 0 and 1 (one group) swaps their weights, not their values' head
    w2 = dict(w, talk=np.eye(4)[[1, 0, 2, 3]])
    o2 = o.copy()
    for t in range(T):
        for a, b in ((0, 1), (1, 0)):
            s = np.array([q[t, b] @ k[j, 0] for j in range(t + 1)]) * 0.7
            p = np.exp(s - s.max())
            o2[t, a] = (p / p.sum()) @ v[:t + 1, 0]
    want2 = (o2.reshape(T, 12) * plain.sigmoid(h @ w["g"].T)) @ w["o"].T
    assert np.abs(plain.talking_attention(h, w2, mx, eps) - want2).max() < 1e-12


def test_plain_router_weights_are_the_softmax_over_the_chosen():
    rng = np.random.default_rng(3)
    w = {"router": rng.normal(0, 1, (5, 7)), "router.b": np.array([0.0, 9.0, 0.0, -9.0, 0.0])}
    h = rng.normal(0, 1, (20, 7))
    chosen, wts, z = plain.route(h, w, {"experts": 5, "top": 2})
    assert (chosen[:, 0] == 1).mean() >= 0.9 and not (chosen == 3).any()       # the bias counts in the choice
    for t in range(20):
        order = np.argsort(-z[t])[:2]
        assert list(chosen[t]) == list(order)
        e = np.exp(z[t, order])
        assert np.allclose(wts[t], e / e.sum())
    _, all_w, z = plain.route(h, w, {"experts": 5, "top": 5})
    e = np.exp(z - z.max(1, keepdims=True))
    assert np.allclose(np.sort(all_w, 1), np.sort(e / e.sum(1, keepdims=True), 1))
