"""The Mavidra decoder in the engine against the plain implementation (tests/plain_mavidra.py): whole prompts,
decoding through cache and states (matrices, convolution inputs, the last token), prompts in portions, unequal
batches, slots and pages used again, long decoding across page borders and windows, the first tokens, greedy
generation through the package's entry point, the command line and trace replay."""
import functools
import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

import plain_mavidra as plain
import mavidra_tiny as st

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
DTYPES = ("float32", "bfloat16")
# bfloat16 runs get routers that their corrections decide (the same experts for every token, weights that vary), so
# that every position can be compared; the 32-bit runs get routers that choose token by token
WEIGHTS = {(name, dtype): st.make_weights(cfg, seed, decided=dtype == "bfloat16")
           for (name, cfg), seed in zip(st.CONFIGS.items(), (31, 32, 33)) for dtype in DTYPES}


@pytest.fixture(scope="module")
def dirs(tmp_path_factory):
    root = tmp_path_factory.mktemp("mavidra")
    return {(name, dtype): st.write_model_dir(root / f"{name}_{dtype}", st.CONFIGS[name], w)
            for (name, dtype), w in WEIGHTS.items()}


@functools.lru_cache(maxsize=None)
def _plain(name, dtype, tokens):
    margins = []
    logits = plain.forward(st.CONFIGS[name], WEIGHTS[name, dtype], list(tokens), margins=margins)
    return logits, (np.min(np.stack(margins), axis=0) if margins else np.full(len(tokens), np.inf))


def plain_logits(name, tokens, dtype="float32"):
    return _plain(name, dtype, tuple(int(t) for t in tokens))[0]


CLOSE_CALL = {"bfloat16": 0.05, "float32": 1e-5}     # in units of a router's scores (sigmoids, and sums of two)


def check_rounded(got, want, what):
    """A bfloat16 run against the plain logits.  Rounding of the activations (8 bits) is passed on by the norms after
    every sub-layer, at single positions at many times its size (a sub-layer's output that is small against its
    neighbours'; the plain implementation shows the same when its activations are disturbed by as much).  So the
    comparison is by position, as a share of the logits' spread with the mean difference taken off: the mean over the
    positions is held tight, and all but a few positions stay within a bound that a wrong key, window or state
    breaks everywhere at once."""
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    assert got.shape == want.shape and np.isfinite(got).all(), what
    spread = max(float(want.std()), 1e-30)
    d = got - want
    e = np.sqrt(((d - d.mean(axis=1, keepdims=True)) ** 2).mean(axis=1)) / spread
    over = int((e > 0.12).sum())
    assert e.mean() <= 0.04 and over <= max(1, int(0.04 * len(e))) and e.max() <= 2.0, \
        f"{what}: by position, mean {e.mean():.4f}, {over} of {len(e)} over 0.12, largest {e.max():.3f} of the spread"


def check(got, name, tokens, dtype, what, rows=None):
    """Holds the engine's logits to the plain ones.  A router's choice between two experts whose logits are closer
    than the rounding of the activations may fall the other way, which is no fault but changes that position and,
    through the states and the cached keys and values of the layers after it, the positions that follow: a run is
    compared up to its first such position (in bfloat16 there is none, by the routers' making)."""
    want, margin = _plain(name, dtype, tuple(int(t) for t in tokens))
    got = np.asarray(got)
    close_calls = np.nonzero(margin <= CLOSE_CALL[dtype])[0]
    upto = int(close_calls[0]) if len(close_calls) else len(margin)
    keep = np.arange(len(margin)) < upto
    if rows is not None:
        want, keep = want[rows], keep[rows]
    assert got.shape == want.shape and np.isfinite(got).all(), what
    got, want = got[keep], want[keep]
    if not len(want):
        return
    if dtype == "bfloat16":
        check_rounded(got, want, what)
        return
    # 32-bit: sums of float32 roundings through norms after every sub-layer and states carried over many tokens
    diff = np.abs(np.asarray(got, np.float64) - want) / max(1.0, float(want.std()))
    assert diff.max() <= 1e-4 and diff.mean() <= 1e-5, f"{what}: max |diff| {diff.max():.3e}, mean {diff.mean():.3e} of the spread"


def some_tokens(name, n, seed):
    return np.random.default_rng(seed).integers(0, st.CONFIGS[name]["vocab"], n).tolist()


_ENGINES: dict = {}


def engine_of(dirs, name, dtype, max_tokens=2048, max_slots=6):
    from alpacca_b200.engine.engine import Engine
    from alpacca_b200.engine.loading import load_model_dir
    key = (name, dtype, max_tokens, max_slots)
    if key not in _ENGINES:
        model = load_model_dir(dirs[name, dtype], dtype, "cuda", max_positions=1024)
        _ENGINES[key] = Engine(model, max_tokens=max_tokens, max_slots=max_slots)
    return _ENGINES[key]


def run(eng, slot, tokens, want=None):
    from alpacca_b200.engine.step import StepEntry
    want = list(range(len(tokens))) if want is None else want
    out = eng.step([StepEntry(slot, tokens, want)]).cpu().numpy()
    eng.wait()
    return out


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(st.CONFIGS))
def test_the_comparisons_reach_every_token(name, dtype):
    """No run of this file is cut short by a router's close call."""
    for n, seed in ((200, 1), (210, 2), (70, 4), (150, 3)):
        _, margin = _plain(name, dtype, tuple(some_tokens(name, n, seed)))
        assert (margin > CLOSE_CALL[dtype]).all(), (name, dtype, n)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(st.CONFIGS))
def test_whole_prompt(dirs, name, dtype):
    eng = engine_of(dirs, name, dtype)
    toks = some_tokens(name, 200, 1)
    s = eng.alloc_slot()
    try:
        check(run(eng, s, toks), name, toks, dtype, f"mavidra {name} whole")
    finally:
        eng.free_slot(s)
    eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(st.CONFIGS))
def test_prompt_then_long_decoding(dirs, name, dtype):
    """50 tokens at once, then 160 one by one: the page borders at 64, 128 and 192 and every window's edge are
    passed while decoding, the states are carried through 160 steps, pages that lie before every window are given
    back on the way, and from the third step on the steps are graph replays."""
    eng = engine_of(dirs, name, dtype)
    toks = some_tokens(name, 210, 2)
    s = eng.alloc_slot()
    try:
        got = [run(eng, s, toks[:50])]
        for p in range(50, 210):
            got.append(run(eng, s, [toks[p]]))
        check(np.concatenate(got), name, toks, dtype, f"mavidra {name} decode")
    finally:
        eng.free_slot(s)
    eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(st.CONFIGS))
def test_token_by_token_from_the_first(dirs, name, dtype):
    eng = engine_of(dirs, name, dtype)
    toks = some_tokens(name, 70, 4)
    s = eng.alloc_slot()
    try:
        check(np.concatenate([run(eng, s, [t]) for t in toks]), name, toks, dtype, f"mavidra {name} token by token")
    finally:
        eng.free_slot(s)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(st.CONFIGS))
@pytest.mark.parametrize("cuts", [(2, 3, 59, 1, 64, 2, 19), (63, 2, 63, 22), (1, 1, 2, 126, 20), (65, 85), (2,) * 40])
def test_prompt_in_portions(dirs, name, dtype, cuts):
    eng = engine_of(dirs, name, dtype)
    toks = some_tokens(name, sum(cuts), 3)
    s = eng.alloc_slot()
    try:
        got, at = [], 0
        for n in cuts:
            got.append(run(eng, s, toks[at:at + n]))
            at += n
        check(np.concatenate(got), name, toks, dtype, f"mavidra {name} portions")
    finally:
        eng.free_slot(s)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(st.CONFIGS))
def test_unequal_batch_against_each_alone(dirs, name, dtype):
    """Four prompts of 1, 70, 33 and 140 tokens in one step, then decoded together; the shorter requests end
    first.  Every request's logits are those of the request alone."""
    from alpacca_b200.engine.step import StepEntry
    eng = engine_of(dirs, name, dtype)
    full = [some_tokens(name, n, 10 + i) for i, n in enumerate((1, 78, 39, 152))]
    first = (1, 70, 33, 140)
    slots = [eng.alloc_slot() for _ in full]
    try:
        got = [[] for _ in full]
        out = eng.step([StepEntry(s, t[:n], list(range(n))) for s, t, n in zip(slots, full, first)]).cpu().numpy()
        at = 0
        for i, n in enumerate(first):
            got[i].append(out[at:at + n])
            at += n
        pos = list(first)
        while any(p < len(t) for p, t in zip(pos, full)):
            live = [i for i in range(len(full)) if pos[i] < len(full[i])]
            out = eng.step([StepEntry(slots[i], [full[i][pos[i]]], [0]) for i in live]).cpu().numpy()
            for j, i in enumerate(live):
                got[i].append(out[j:j + 1])
                pos[i] += 1
        eng.wait()
        for i, t in enumerate(full):
            check(np.concatenate(got[i]), name, t, dtype, f"mavidra {name} batch row {i}")
    finally:
        for s in slots:
            eng.free_slot(s)
    eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["a", "c"])
def test_slots_and_pages_used_again(dirs, name, dtype):
    """A cache of five pages and two slots: every new sequence gets a slot and pages that another one has just
    given back, with its keys still in the pages and its matrices, convolution inputs and last token still in the
    states' rows."""
    eng = engine_of(dirs, name, dtype, max_tokens=320, max_slots=2)
    for k, n in enumerate((130, 100, 3, 128, 65)):
        toks = some_tokens(name, n, 20 + k)
        s = eng.alloc_slot()
        other = eng.alloc_slot() if n <= 100 else None
        try:
            cut = max(1, n - 3)
            got = [run(eng, s, toks[:cut])]
            if other is not None:
                run(eng, other, some_tokens(name, 40, 99))       # a neighbour that writes pages and states too
            for p in range(cut, n):
                got.append(run(eng, s, [toks[p]]))
            check(np.concatenate(got), name, toks, dtype, f"mavidra reuse {k}")
        finally:
            eng.free_slot(s)
            if other is not None:
                eng.free_slot(other)
        eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(st.CONFIGS))
def test_first_tokens(dirs, name, dtype):
    eng = engine_of(dirs, name, dtype)
    toks = some_tokens(name, 3, 30)
    for cuts in ((3,), (1, 1, 1), (1, 2), (2, 1)):
        s = eng.alloc_slot()
        try:
            got, at = [], 0
            for n in cuts:
                got.append(run(eng, s, toks[at:at + n]))
                at += n
            check(np.concatenate(got), name, toks, dtype, f"mavidra {name} first tokens")
        finally:
            eng.free_slot(s)


def test_wanted_places_only(dirs):
    eng = engine_of(dirs, "b", "float32")
    toks = some_tokens("b", 90, 31)
    want = [0, 17, 63, 64, 89]
    s = eng.alloc_slot()
    try:
        check(run(eng, s, toks, want), "b", toks, "float32", "mavidra wanted places", rows=want)
    finally:
        eng.free_slot(s)


@pytest.mark.parametrize("name", ["a", "b"])
def test_the_stream_after_every_layer(dirs, name):
    from alpacca_b200.engine.step import StepEntry
    eng = engine_of(dirs, name, "float32")
    toks = some_tokens(name, 40, 32)
    trace = []
    plain.forward(st.CONFIGS[name], WEIGHTS[name, "float32"], toks, trace=trace)
    seen = []
    layers = eng.model.spec.layers
    originals = [blk.forward for blk in layers]

    def spy(blk, original):
        def forward(stream, ctx, cache, write_cache=True):
            original(stream, ctx, cache, write_cache)
            assert stream.delta is None           # the norm after a sub-layer leaves nothing waiting
            seen.append(stream.residual[:ctx.n_tokens].double().cpu().numpy())
        return forward
    s = eng.alloc_slot()
    try:
        for blk, original in zip(layers, originals):
            blk.forward = spy(blk, original)
        eng.forget_graphs()
        eng.step([StepEntry(s, toks, [])])
        eng.wait()
    finally:
        for blk in layers:
            del blk.forward
        eng.free_slot(s)
        eng.forget_graphs()
    assert len(seen) == len(trace) == len(st.CONFIGS[name]["layers"])
    for i, (a, b) in enumerate(zip(seen, trace)):
        assert np.abs(a - b).max() <= 1e-4 * max(1.0, np.abs(b).max()), f"stream after layer {i}"


def plain_greedy(name, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(np.argmax(plain_logits(name, toks)[-1])))
    return toks[len(prompt):]


@pytest.mark.parametrize("graphs", [True, False])
@pytest.mark.parametrize("name", ["a", "c"])
def test_greedy_generation_through_the_entry_point(dirs, name, graphs):
    """`Model.load` + `generate` (the scheduler, the graph decoder with its padded rows, the device sampler)
    give the plain implementation's greedy tokens, for prompts of unequal lengths that end at different steps."""
    from alpacca_b200.api import Model, generate
    from alpacca_b200.sampling import SamplerParams
    model = Model.load(dirs[name, "float32"], n_ctx=256, dtype="float32", max_batch=4, progress=False)
    if not graphs:
        model.use_graphs = False
    prompts = [some_tokens(name, n, 40 + i) for i, n in enumerate((5, 70, 1))]
    budgets = 12
    res = generate(model, prompts, SamplerParams.greedy(), n_predict=budgets)
    for p, r in zip(prompts, res):
        assert r.token_ids == plain_greedy(name, p, budgets)
    again = generate(model, prompts[::-1], SamplerParams.greedy(), n_predict=4)      # the same slots once more
    for p, r in zip(prompts[::-1], again):
        assert r.token_ids == plain_greedy(name, p, 4)


def test_generation_in_bfloat16_runs(dirs):
    from alpacca_b200.api import Model, generate
    from alpacca_b200.sampling import SamplerParams
    model = Model.load(dirs["b", "bfloat16"], n_ctx=256, dtype="bfloat16", max_batch=4, progress=False)
    res = generate(model, [some_tokens("b", 30, 50), some_tokens("b", 2, 51)], SamplerParams(temperature=0.8, seed=3),
                   n_predict=20)
    assert all(len(r.token_ids) == 20 and all(0 <= t < st.CONFIGS["b"]["vocab"] for t in r.token_ids) for r in res)


@pytest.mark.parametrize("dtype", DTYPES)
def test_trace_replay(dirs, dtype, tmp_path):
    name = "a"
    a, b = some_tokens(name, 70, 60), some_tokens(name, 9, 61)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:66], "want": [0, 65]},
                                     {"id": "b", "tokens": b[:7], "want": [6]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[66:67], "want": [0]},
                                     {"id": "b", "tokens": b[7:8], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": a[67:68], "want": [0]},
                                     {"id": "b", "tokens": b[8:9], "want": [0]}], "end": ["b"]},
             {"step": 3, "entries": [{"id": "a", "tokens": a[68:70], "want": [1]}], "end": ["a"]}]
    out = tmp_path / "out"
    proc = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(dirs[name, dtype]), "--dtype", dtype,
                           "--out", str(out), "--max-tokens", "256"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [ln for ln in proc.stdout.splitlines() if ln.startswith("done")] == [f"done {i}" for i in range(4)]
    V = st.CONFIGS[name]["vocab"]
    pa, pb = plain_logits(name, a, dtype), plain_logits(name, b, dtype)
    want = {0: np.stack([pa[0], pa[65], pb[6]]), 1: pa[66:67], 2: np.stack([pa[67], pb[8]]), 3: pa[69:70]}
    for i, w in want.items():
        got = np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, V)
        if dtype == "bfloat16":
            check_rounded(got, w, "mavidra trace replay")
        else:
            assert np.abs(got - w).max() <= 1e-4 * max(1.0, float(w.std()))


def test_run_command(dirs):
    """`python -m alpacca_b200 run` with a Mavidra folder: two prompts as one batch, greedy, in 32-bit."""
    name = "c"
    prompts = [some_tokens(name, 6, 70), some_tokens(name, 2, 71)]
    text = " / ".join(" ".join(map(str, p)) for p in prompts)
    proc = subprocess.run([sys.executable, "-m", "alpacca_b200", "run", str(dirs[name, "float32"]), text, "--temp", "0",
                           "--repeat-penalty", "1.0", "--n-predict", "5", "--dtype", "float32", "--ctx", "64"],
                          capture_output=True, text=True, timeout=600, cwd=str(ROOT))
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = [ln for ln in proc.stdout.splitlines() if ln.strip()]
    assert [[int(t) for t in ln.split()] for ln in lines] == [plain_greedy(name, p, 5) for p in prompts]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["b", "c"])
def test_prompt_steps_replayed_from_their_graph(dirs, name, dtype):
    """Five prompt steps of one shape (two prompts of 70 and 9 tokens on empty slots): the second is captured, the
    later ones are replays with other tokens, slots and pages, and every one gives the plain logits."""
    from alpacca_b200.engine.step import StepEntry
    eng = engine_of(dirs, name, dtype)
    held = eng.alloc_slot()          # shifts the slots of the later rounds
    for k in range(5):
        a, b = some_tokens(name, 70, 300 + k), some_tokens(name, 9, 320 + k)
        if k == 3:
            eng.free_slot(held)
            held = None
        sa, sb = eng.alloc_slot(), eng.alloc_slot()
        out = eng.step([StepEntry(sa, a, list(range(70))), StepEntry(sb, b, list(range(9)))]).cpu().numpy()
        eng.wait()
        check(out[:70], name, a, dtype, f"mavidra {name} replayed prompt step {k}")
        check(out[70:], name, b, dtype, f"mavidra {name} replayed prompt step {k}, second prompt")
        eng.free_slot(sa)
        eng.free_slot(sb)
    assert len(eng._graphs) >= 1
