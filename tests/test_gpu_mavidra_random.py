"""Mavidra configurations drawn at random from fixed seeds (`mavidra_tiny.random_config`): 2 to 6 layers in any
order; gated linear attention of 1 to 5 heads with key sizes 8 to 136 and decay ranks 1 to 16; latent attention with
windows of 3 to 100 tokens or none, some layers reading an earlier layer's cache with a window of their own; attention
of 1 to 9 heads on 1 to 3 key/value heads beside a delta rule with convolutions over 1 to 6 tokens; rotations over all,
half or none of a vector; 1 to 20 experts in 1 to 4 groups of which some or all are kept; layers without a
feed-forward; widths that are no multiples of 8, 4 or 2; hash tables of 7 to 509 rows with multipliers up to a
million.  Each whole beside another request, in portions, and with its last tokens one by one, in both precisions;
in bfloat16 the routers are made so that their corrections decide."""
import functools

import numpy as np
import pytest

import plain_mavidra as plain
import mavidra_tiny as st

pytestmark = pytest.mark.gpu

SEEDS = list(range(16))


@functools.lru_cache(maxsize=None)
def model_of(seed, dtype):
    cfg = st.random_config(seed)
    return cfg, st.make_weights(cfg, 700 + seed, decided=dtype == "bfloat16")


@pytest.fixture(scope="module")
def root(tmp_path_factory):
    return tmp_path_factory.mktemp("mavidra_random")


def check(got, want, margin, dtype, what):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    assert got.shape == want.shape and np.isfinite(got).all(), what
    close_calls = np.nonzero(margin <= (0.05 if dtype == "bfloat16" else 1e-5))[0]
    upto = int(close_calls[0]) if len(close_calls) else len(want)
    assert upto >= len(want) // 2 or dtype == "float32", f"{what}: the routers of this seed decide too little"
    d = np.abs(got - want)[:upto]
    if not upto:
        return
    spread = max(float(want.std()), 1e-30)
    if dtype == "float32":
        assert d.max() <= 1e-4 * max(1.0, spread) and d.mean() <= 1e-5 * max(1.0, spread), \
            f"{what}: max |diff| {d.max():.3e}, mean {d.mean():.3e}"
        return
    # bfloat16: by position, as in tests/test_gpu_mavidra.py (`check_rounded` there says why)
    diff = (got - want)[:upto]
    e = np.sqrt(((diff - diff.mean(axis=1, keepdims=True)) ** 2).mean(axis=1)) / spread
    over = int((e > 0.12).sum())
    assert e.mean() <= 0.04 and over <= max(1, int(0.04 * len(e))) and e.max() <= 2.0, \
        f"{what}: by position, mean {e.mean():.4f}, {over} of {len(e)} over 0.12, largest {e.max():.3f} of the spread"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", SEEDS)
def test_random_configuration(root, seed, dtype):
    from alpacca_b200.engine.engine import Engine
    from alpacca_b200.engine.loading import load_model_dir
    from alpacca_b200.engine.step import StepEntry
    cfg, weights = model_of(seed, dtype)
    folder = st.write_model_dir(root / f"m{seed}_{dtype}", cfg, weights)
    eng = Engine(load_model_dir(folder, dtype, "cuda", max_positions=512), max_tokens=1024, max_slots=3)
    rng = np.random.default_rng(seed)
    toks = rng.integers(0, cfg["vocab"], 150).tolist()
    other = rng.integers(0, cfg["vocab"], 30).tolist()

    def plain_of(t):
        margins = []
        lg = plain.forward(cfg, weights, t, margins=margins)
        return lg, (np.min(np.stack(margins), axis=0) if margins else np.full(len(t), np.inf))
    (want, margin), (want_other, margin_other) = plain_of(toks), plain_of(other)

    def run(entries):
        out = eng.step([StepEntry(s, t, list(range(len(t)))) for s, t in entries]).cpu().numpy()
        eng.wait()
        return out
    a, b = eng.alloc_slot(), eng.alloc_slot()
    both = run([(b, other), (a, toks)])
    check(both[:30], want_other, margin_other, dtype, f"seed {seed}: the short request of a batch")
    check(both[30:], want, margin, dtype, f"seed {seed}: whole")
    eng.free_slot(a)
    eng.free_slot(b)
    a = eng.alloc_slot()
    got = [run([(a, toks[:3])]), run([(a, toks[3:5])]), run([(a, toks[5:70])]), run([(a, toks[70:110])])]
    got += [run([(a, [t])]) for t in toks[110:]]
    check(np.concatenate(got), want, margin, dtype, f"seed {seed}: in portions and token by token")
    eng.free_slot(a)
    eng.cache.check()
