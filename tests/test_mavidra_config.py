"""The Mavidra decoder without a GPU: configuration faults, tensor names and shapes, the schedule and its cache
entries, sizes read from a checkpoint's tensor shapes, and the plain implementation against hand-made cases."""
import copy

import numpy as np
import pytest
import torch

import mavidra_tiny as mt
import plain_mavidra as plain
from alpacca_b200.config import ConfigError, config_from_dict
from alpacca_b200.engine.loading import build_model
from alpacca_b200.parts.base import KVSpec, StateSpec


@pytest.mark.parametrize("name", list(mt.CONFIGS))
def test_tensor_names_and_shapes(name):
    model = build_model(copy.deepcopy(mt.CONFIGS[name]), torch.float32, "cpu", 256)
    specs = {s.name: tuple(s.shape) for s in model.param_specs() if not s.absent}
    assert specs == mt.tensor_shapes(mt.CONFIGS[name])


def test_random_configurations_are_valid_and_differ():
    seen = set()
    for seed in range(40):
        cfg = mt.random_config(seed)
        model = build_model(copy.deepcopy(cfg), torch.float32, "cpu", 128)
        specs = {s.name: tuple(s.shape) for s in model.param_specs() if not s.absent}
        assert specs == mt.tensor_shapes(cfg), seed
        seen.add(tuple(layer["type"] for layer in cfg["layers"]))
    assert len(seen) > 20


def test_schedule_and_cache_entries():
    model = build_model(copy.deepcopy(mt.TINY_A), torch.float32, "cpu", 256)
    runs = model.spec.schedule
    assert [r.layer for r in runs] == [0, 1, 2, 3] and [r.reads_entry_of for r in runs] == [None, None, None, 0]
    specs = model.cache_entry_specs()
    # the first layer caches latent rows for its own window of 70 and for the reader's of 33: the wider one
    assert specs[0] == KVSpec(1, 28, 70, values=False)
    assert specs[1] == StateSpec((2, 12, 20), torch.float32)
    assert specs[2] == KVSpec(2, 16, None, value_heads=2, value_dim=24)
    assert specs[3] == StateSpec((6, 8, 12), torch.float32) and specs[4] == StateSpec((2, 2 * 3 * 8 + 6 * 12), torch.float32)
    assert specs[5] == StateSpec((1,), torch.int32)            # the embedding keeps each sequence's last token
    assert model.entries_of_run == [[0], [1], [2, 3, 4], [0]] and model.embedding_entry == 5
    # a reader with the wider window widens what the owner keeps; a reader without a window makes it keep everything
    b = build_model(copy.deepcopy(mt.TINY_B), torch.float32, "cpu", 256)
    assert b.cache_entry_specs()[4] == KVSpec(1, 32, 130, values=False)
    cfg = copy.deepcopy(mt.TINY_B)
    del cfg["layers"][3]["mixer"]["mask"]
    assert build_model(cfg, torch.float32, "cpu", 256).cache_entry_specs()[4] == KVSpec(1, 32, None, values=False)


def test_rank_from_tensor_shapes():
    cfg = copy.deepcopy(mt.TINY_A)
    del cfg["layers"][1]["mixer"]["rank"]
    parsed = config_from_dict(cfg)
    with pytest.raises(ValueError, match="rank"):
        build_model(parsed, torch.float32, "cpu", 64)
    done = parsed.with_shapes({"l1.mix.a1": (5, 40), "l0.mix.dq": (24, 40)})
    assert done.layers[1]["mixer"]["rank"] == 5 and "rank" not in parsed.layers[1]["mixer"]
    specs = {s.name: tuple(s.shape) for s in build_model(done, torch.float32, "cpu", 64).param_specs()}
    assert specs["l1.mix.a2"] == (24, 5)


@pytest.mark.parametrize("change,word", [
    (lambda c: c["layers"][0].update(type="attention"), "not supported"),
    (lambda c: c["layers"][1]["mixer"].update(tau=0.0), "tau"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=2), "kv_from"),
    (lambda c: c["layers"][3]["mixer"].update(kv_rank=24), "kv_rank"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=10), "dims"),
    (lambda c: c["layers"][2]["mixer"]["left"].update(kv_heads=3), "share"),
    (lambda c: c["layers"][2]["mixer"]["right"].pop("conv"), "conv"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=5), "chosen"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=4), "equal groups"),
    (lambda c: c["embedding"].pop("scale"), "scale"),
    (lambda c: c["embedding"]["bigram"].pop("buckets"), "buckets"),
    (lambda c: c.pop("width"), "width"),
])
def test_faults_are_named(change, word):
    cfg = copy.deepcopy(mt.TINY_A)
    change(cfg)
    with pytest.raises(ConfigError, match=word):
        config_from_dict(cfg)


# -- the plain implementation against cases made by hand -------------------------------------------------------
def test_plain_layer_norm_and_embedding():
    x = np.array([[1.0, 2.0, 3.0, 6.0]])
    y = plain.layer_norm(x, np.array([1.0, 1.0, 2.0, 1.0]), np.array([0.0, 0.5, 0.0, 0.0]), 0.0)
    sd = np.sqrt(np.mean((x - 3.0) ** 2))
    assert np.allclose(y, [[-2 / sd, -1 / sd + 0.5, 0.0, 3 / sd]])
    W = {"embed": np.arange(12.0).reshape(6, 2), "bigram": np.arange(100.0, 112.0).reshape(6, 2)}
    emb = {"scale": 2.0, "bigram": {"buckets": 5, "mul_prev": 3, "mul_cur": 4}}
    got = plain.embed([4, 1, 5], W, emb)
    rows = [5, (4 * 3 + 1 * 4) % 5, (1 * 3 + 5 * 4) % 5]
    assert np.allclose(got, W["embed"][[4, 1, 5]] * 2.0 + W["bigram"][rows])


def test_plain_turns_keep_lengths_and_pairs():
    rng = np.random.default_rng(0)
    x = rng.normal(size=(5, 2, 8))
    rot = {"base": 100.0, "dims": 4}
    for inter in (False, True):
        y = plain.turn(x, np.arange(5), rot, inter)
        assert np.allclose(y[..., 4:], x[..., 4:]) and np.allclose(y[0], x[0])
        assert np.allclose((y ** 2).sum(-1), (x ** 2).sum(-1))
    a = np.cos(3.0), np.sin(3.0)
    y = plain.turn(x, np.arange(5), rot, True)
    assert np.allclose(y[3, 0, 0], x[3, 0, 0] * a[0] - x[3, 0, 1] * a[1])
    y = plain.turn(x, np.arange(5), rot, False)
    assert np.allclose(y[3, 0, 0], x[3, 0, 0] * a[0] - x[3, 0, 2] * a[1])


def test_plain_attention_window_and_sink():
    rng = np.random.default_rng(1)
    q, k, v = rng.normal(size=(6, 2, 4)), rng.normal(size=(6, 1, 4)), rng.normal(size=(6, 1, 3))
    full = plain.softmax_attention(q, k, v, 0.5)
    assert np.allclose(full[0, :, :], v[0, 0])
    win = plain.softmax_attention(q, k, v, 0.5, window=2)
    s = np.array([q[4, 1] @ k[3, 0], q[4, 1] @ k[4, 0]]) * 0.5
    p = np.exp(s) / np.exp(s).sum()
    assert np.allclose(win[4, 1], p[0] * v[3, 0] + p[1] * v[4, 0])
    # a sink far above the scores takes all the weight; far below, none
    assert np.abs(plain.softmax_attention(q, k, v, 0.5, sink=np.array([50.0, 50.0]))).max() < 1e-15
    assert np.allclose(plain.softmax_attention(q, k, v, 0.5, sink=np.array([-80.0, -80.0])), full)


def test_plain_conv_and_delta_rule():
    x = np.arange(1.0, 6.0)[:, None] * np.array([[1.0, 10.0]])
    taps = np.array([[0.5, 0.0, 1.0], [1.0, 1.0, 1.0]])
    y = plain.short_conv(x, taps)
    assert np.allclose(y[:, 0], [1, 2, 3.5, 5, 6.5]) and np.allclose(y[:, 1], [10, 30, 60, 90, 120])
    # one head, keys that are unit vectors: writing the same key twice with beta 1 and no decay replaces the value
    S = np.zeros((2, 2))
    k = np.array([1.0, 0.0])
    for v in (np.array([3.0, 4.0]), np.array([-1.0, 2.0])):
        u = v - S.T @ k
        S = S + np.outer(k, u)
    assert np.allclose(S.T @ k, [-1.0, 2.0])


def test_plain_router_groups_and_negative_scores():
    h = np.eye(4)[:1]
    # 6 experts in 3 groups of 2, 2 groups kept, 2 chosen.  Corrections push every choice score of group 0 below zero
    # although its plain scores are the largest: the choice must not fall back on them.
    w = {"router": np.array([[4.0, 0, 0, 0], [3.0, 0, 0, 0], [0.2, 0, 0, 0], [0.1, 0, 0, 0], [-1.0, 0, 0, 0], [0.0, 0, 0, 0]]),
         "correction": np.array([-5.0, -5.0, 0.0, 0.0, 0.3, 0.0])}
    chosen, wts, _ = plain.route(h, w, {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 2}})
    s = 1.0 / (1.0 + np.exp(-w["router"][:, 0]))
    assert sorted(chosen[0]) == [2, 4] and np.allclose(sorted(wts[0]), sorted(s[[2, 4]]))
    # with only one group kept and three wanted from it ... the struck groups never come back
    chosen, _, _ = plain.route(h, w, {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 1}})
    assert sorted(chosen[0]) == [2, 3]
    # a group's score is the sum of its two largest choice scores, not its largest
    w2 = {"router": np.zeros((6, 4)), "correction": np.array([0.9, -0.9, 0.5, 0.5, 0.0, 0.0])}
    chosen, _, _ = plain.route(h, w2, {"experts": 6, "top": 1, "groups": {"count": 3, "keep": 1}})
    assert chosen[0, 0] == 2


def test_plain_gla_is_a_decayed_sum():
    rng = np.random.default_rng(3)
    E, H, D, V, T = 6, 1, 3, 2, 5
    mx = {"heads": H, "dim": D, "vdim": V, "tau": 2.0}
    w = {n: rng.normal(size=s) for n, s in (("q", (D, E)), ("k", (D, E)), ("v", (V, E)), ("g", (V, E)), ("o", (E, V)),
                                           ("a1", (2, E)), ("a2", (D, 2)), ("a2.b", (D,)))}
    w["norm"] = np.ones(V)
    h = rng.normal(size=(T, E))
    q, k, v = h @ w["q"].T * D ** -0.5, h @ w["k"].T, h @ w["v"].T
    a = (1.0 / (1.0 + np.exp(-((h @ w["a1"].T) @ w["a2"].T + w["a2.b"])))) ** 0.5
    o = np.zeros((T, V))
    for t in range(T):
        for s in range(t + 1):
            o[t] += ((q[t] * k[s] * np.prod(a[s + 1:t + 1], axis=0)).sum()) * v[s]
    want = (plain.rms(o, 1e-6) * (h @ w["g"].T) / (1 + np.exp(-(h @ w["g"].T)))) @ w["o"].T
    assert np.allclose(plain.gla(h, w, mx, 1e-6), want)
