"""Each mechanism of the Mavidra decoder alone, against its function in tests/plain_mavidra.py: the layer norm and
the kernel that norms a sub-layer's output into the stream, the embedding with its table of token pairs, gated linear
attention, the gated delta rule with its convolutions, the attention with a sink and a gate per head, latent
attention with a window (also read by a second layer with a window of its own), and the router with sigmoid scores,
a correction and groups.  Sizes differ from test to test; inputs are made so that faults show."""
import numpy as np
import pytest
import torch

import plain_mavidra as plain
from helpers import PartHarness, load_part

pytestmark = pytest.mark.gpu

TOL = {"float32": (2e-4, 2e-5), "bfloat16": (0.2, 0.02)}      # (largest, mean) |difference| as shares of the spread
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
DTYPES = ["float32", "bfloat16"]


def close(got, want, dtype, what, tol=None):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    assert got.shape == want.shape and np.isfinite(got).all(), what
    spread = max(float(want.std()), 1e-30)
    d = np.abs(got - want) / spread
    big, mean = tol or TOL[dtype]
    assert d.max() <= big and d.mean() <= mean, f"{what}: max {d.max():.3e} mean {d.mean():.3e} of the spread"


def opts_of(dtype, max_positions=1024):
    from alpacca_b200.parts import BuildOptions
    return BuildOptions(dtype=DT[dtype], device="cuda", max_positions=max_positions)


def hidden(rng, n, width, dtype):
    """Activations [n, width] that both precisions hold exactly."""
    x = torch.from_numpy(rng.normal(0.0, 1.0, (n, width)).astype(np.float32)).to(torch.bfloat16)
    return x.to(DT[dtype]).cuda().contiguous(), x.double().numpy()


def as_input(x64, dtype):
    x = torch.from_numpy(np.asarray(x64, np.float32)).to(torch.bfloat16)
    return x.to(DT[dtype]).cuda().contiguous(), x.double().numpy()


def short(weights, prefix):
    return {k[len(prefix) + 1:]: v for k, v in weights.items() if k.startswith(prefix + ".")}


def views_of(hs, ctx, n):
    views = [hs.cache.entry_view(e, ctx.block_tables) for e in range(n)]
    return views[0] if n == 1 else views


def feed(part, hs, slot, x, cuts, n_entries=1, first_entry=0, write_cache=True):
    """Runs `x` through a mixer in portions; returns the outputs as one array."""
    out, at = [], 0
    for n in cuts:
        ctx = hs.step([(slot, n)])
        views = [hs.cache.entry_view(first_entry + e, ctx.block_tables) for e in range(n_entries)]
        out.append(part.forward(x[at:at + n].contiguous(), ctx, views[0] if n_entries == 1 else views,
                                write_cache).float().cpu().numpy())
        hs.done()
        at += n
    assert at == x.shape[0]
    return np.concatenate(out)


# ---------------------------------------------------------------------------------------------------------------
# layer norm, and the kernel after a sub-layer
# ---------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [37, 256, 1000, 4096, 13000])
def test_layer_norm_and_the_kernel_after_a_sublayer(dtype, width):
    from alpacca_b200 import ops
    rng = np.random.default_rng(width)
    T, eps, mult = 9, 1e-5, 0.35
    x64 = rng.normal(2.0, 3.0, (T, width))          # a mean far from zero: the variance is taken about it
    w, b, w2, b2 = (rng.normal(1.0, 0.4, width), rng.normal(0.0, 0.5, width), rng.normal(1.0, 0.4, width),
                    rng.normal(0.0, 0.5, width))
    dev = lambda a: torch.from_numpy(np.asarray(a, np.float32)).cuda().contiguous()      # noqa: E731
    x = dev(x64)
    x64 = x.double().cpu().numpy()
    out = torch.empty((T, width), dtype=DT[dtype], device="cuda")
    ops.layer_norm(x, None, dev(w), dev(b), eps, out)
    want = plain.layer_norm(x64, dev(w).double().cpu().numpy(), dev(b).double().cpu().numpy(), eps)
    close(out.float().cpu().numpy(), want, dtype, "layer norm", tol=(2e-5, 2e-6) if dtype == "float32" else (0.02, 0.003))
    rows = torch.tensor([7, 0, 3], dtype=torch.int32, device="cuda")
    picked = torch.empty((3, width), dtype=DT[dtype], device="cuda")
    ops.layer_norm(x, None, dev(w), dev(b), eps, picked, rows=rows)
    assert torch.equal(picked, out[[7, 0, 3]]) and torch.equal(x, dev(x64))
    for two in (False, True):
        a, a64 = hidden(rng, T, width, dtype)
        c, c64 = hidden(rng, T, width, dtype)
        res = dev(x64)
        nxt = torch.empty((T, width), dtype=DT[dtype], device="cuda")
        more = {"b": c, "ca": 1.25, "cb": -0.5} if two else {}
        ops.post_layer_norm_add(res, a, dev(w), dev(b), eps, mult, next_weight=dev(w2), next_bias=dev(b2), out=nxt, **more)
        y = 1.25 * a64 - 0.5 * c64 if two else a64
        f64 = lambda v: dev(v).double().cpu().numpy()       # noqa: E731
        want_x = x64 + mult * plain.layer_norm(y, f64(w), f64(b), eps)
        close(res.cpu().numpy(), want_x, "float32", "the stream after a sub-layer", tol=(2e-5, 2e-6))
        close(nxt.float().cpu().numpy(), plain.layer_norm(want_x, f64(w2), f64(b2), eps), dtype, "the next norm",
              tol=(3e-5, 3e-6) if dtype == "float32" else (0.02, 0.003))


# ---------------------------------------------------------------------------------------------------------------
# the embedding with its pair table
# ---------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("buckets,mul_prev,mul_cur", [(53, 31, 7), (1, 5, 5), (509, 1000003, 131)])
def test_embedding_with_pairs(dtype, buckets, mul_prev, mul_cur):
    """Two sequences in portions down to one token: the pair of a portion's first token is made with the LAST token
    of the portion before, which the sequence keeps; a slot that is used again starts with the first-token row."""
    from alpacca_b200.engine.step import StepEntry
    from alpacca_b200.parts import PairTable, TokenEmbedding
    V, E, scale = 90, 24, 3.5
    opts = opts_of(dtype)
    emb = TokenEmbedding(opts, V, E, "embed", weight_suffix="", scale=scale,
                         pairs=PairTable(opts, buckets, E, mul_prev, mul_cur, "bigram"))
    w = load_part(emb, seed=buckets, dtype=dtype, std=1.0)
    cfg = {"scale": scale, "bigram": {"buckets": buckets, "mul_prev": mul_prev, "mul_cur": mul_cur}}
    rng = np.random.default_rng(buckets)
    hs = PartHarness([emb.cache_spec()], dtype, max_slots=3)

    def step(seqs):
        entries = [StepEntry(s, t, []) for s, t in seqs]
        hs.cache.reserve([(s, len(t)) for s, t in seqs])
        ctx = hs.builder.build(entries, [hs.cache.length(s) for s, _ in seqs], hs.cache)
        out = emb.forward(ctx.tokens, ctx.n_tokens, ctx=ctx, cache=hs.cache.entry_view(0, ctx.block_tables)).cpu().numpy()
        hs.cache.commit([(s, len(t)) for s, t in seqs])
        return out
    a, b = rng.integers(0, V, 40).tolist(), rng.integers(0, V, 11).tolist()
    wa, wb = plain.embed(a, w, cfg), plain.embed(b, w, cfg)
    s0, s1 = hs.cache.alloc_slot(), hs.cache.alloc_slot()
    got_a, got_b = [], []
    first = step([(s0, a[:7]), (s1, b[:1])])
    got_a.append(first[:7]), got_b.append(first[7:])
    second = step([(s1, b[1:3]), (s0, a[7:8])])
    got_b.append(second[:2]), got_a.append(second[2:])
    for lo, hi in ((8, 9), (9, 30), (30, 32), (32, 40)):
        got_a.append(step([(s0, a[lo:hi])]))
    got_b.append(step([(s1, b[3:])]))
    assert np.abs(np.concatenate(got_a) - wa).max() <= 1e-5 and np.abs(np.concatenate(got_b) - wb).max() <= 1e-5
    hs.cache.free_slot(s0)
    s2 = hs.cache.alloc_slot()
    assert s2 == s0 and np.abs(step([(s2, b)]) - wb).max() <= 1e-5


# ---------------------------------------------------------------------------------------------------------------
# gated linear attention
# ---------------------------------------------------------------------------------------------------------------
def gla_part(dtype, width, H, D, V, rank, tau, eps):
    from alpacca_b200.parts import GatedLinearAttention
    part = GatedLinearAttention(opts_of(dtype), width, H, D, V, rank, tau, eps, "m", out_dtype=torch.float32)
    return part, {"heads": H, "dim": D, "vdim": V, "tau": tau}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,D,V,rank,tau", [(2, 16, 24, 4, 2.0), (1, 24, 40, 1, 16.0), (3, 64, 20, 16, 1.0), (2, 128, 36, 8, 4.0),
                                            (1, 7, 33, 3, 8.0), (5, 32, 32, 5, 16.0), (1, 200, 130, 12, 3.0), (4, 33, 9, 2, 1.5)])
def test_gated_linear_attention(dtype, H, D, V, rank, tau):
    """Two sequences side by side, fed in portions of unequal sizes down to one token; the state is carried from step
    to step; a slot that is used again starts from zero."""
    width, eps = 56, 1e-5
    part, mx = gla_part(dtype, width, H, D, V, rank, tau, eps)
    w = short(load_part(part, seed=H * 100 + D, dtype=dtype, std=0.25), "m")
    assert set(w) == {"q", "k", "v", "g", "o", "norm", "a1", "a2", "a2.b"}
    rng = np.random.default_rng(D)
    xs = [hidden(rng, n, width, dtype) for n in (75, 31)]
    want = [plain.gla(x64, w, mx, eps) for _, x64 in xs]
    hs = PartHarness([part.cache_spec()], dtype, max_slots=3)
    s0, s1 = hs.cache.alloc_slot(), hs.cache.alloc_slot()
    ctx = hs.step([(s0, 20), (s1, 9)])
    first = part.forward(torch.cat([xs[0][0][:20], xs[1][0][:9]]).contiguous(), ctx, views_of(hs, ctx, 1)).float().cpu().numpy()
    hs.done()
    got0 = np.concatenate([first[:20], feed(part, hs, s0, xs[0][0][20:], (1, 2, 17, 1, 34))])
    got1 = np.concatenate([first[20:], feed(part, hs, s1, xs[1][0][9:], (2, 2, 1, 17))])
    close(got0, want[0], dtype, "gated linear attention, first sequence")
    close(got1, want[1], dtype, "gated linear attention, second sequence")
    hs.cache.free_slot(s0)
    s2 = hs.cache.alloc_slot()
    assert s2 == s0
    close(feed(part, hs, s2, xs[1][0], (31,)), want[1], dtype, "gated linear attention, a slot used again")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("decode", [False, True])
def test_gated_linear_attention_keeps_and_forgets_by_its_decay(dtype, decode):
    """One early token carries a large value; six hundred tokens later the output still shows it in the head whose
    decay is 1 to rounding (a bias of +30 under the sigmoid), and has forgotten it in the head that halves its state
    with every token.  The answer with the early token differs from the one without."""
    width, eps, T = 32, 1e-6, 600
    part, mx = gla_part(dtype, width, 2, 16, 16, 2, 1.0, eps)
    w = short(load_part(part, seed=5, dtype=dtype, std=0.2), "m")
    bias = np.concatenate([np.full(16, 30.0), np.zeros(16)]).astype(np.float32)
    part.b_a2.copy_(torch.from_numpy(bias).cuda())
    part.w_a2.zero_()          # (kept transposed by the part)
    w["a2.b"], w["a2"] = bias.astype(np.float64), np.zeros_like(w["a2"])
    rng = np.random.default_rng(2)
    x64 = rng.normal(0.0, 0.3, (T, width))
    x64[3] *= 40.0
    x, x64 = as_input(x64, dtype)
    want = plain.gla(x64, w, mx, eps)
    without = x64.copy()
    without[3] = 0.0
    assert np.abs(plain.gla(without, w, mx, eps)[-1] - want[-1]).max() > 0.3 * want.std()
    hs = PartHarness([part.cache_spec()], dtype)
    s = hs.cache.alloc_slot()
    got = feed(part, hs, s, x, (T - 40,) + (1,) * 40 if decode else (T,))
    close(got, want, dtype, "a far token in the state")


# ---------------------------------------------------------------------------------------------------------------
# the gated delta rule
# ---------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,D,V,taps", [(4, 2, 16, 24, 4), (2, 2, 24, 40, 1), (6, 1, 64, 20, 2), (2, 1, 128, 36, 5),
                                          (3, 3, 7, 33, 3), (1, 1, 200, 130, 4), (8, 4, 32, 8, 6)])
def test_gated_delta_rule(dtype, H, G, D, V, taps):
    """Portions of one, two and three tokens put a portion's border inside every convolution's reach; the convolution's
    last inputs and the matrix per head are carried from step to step, for two sequences side by side."""
    from alpacca_b200.parts import GatedDeltaRule
    width, eps = 48, 1e-5
    part = GatedDeltaRule(opts_of(dtype), width, H, G, D, V, taps, eps, "m", out_dtype=torch.float32)
    mx = {"heads": H, "kv_heads": G, "dim": D, "vdim": V, "conv": taps}
    w = short(load_part(part, seed=H * 10 + taps, dtype=dtype, std=0.3), "m")
    assert {"q.conv", "k.conv", "v.conv", "A_log", "dt_bias", "b", "a", "norm"} <= set(w)
    rng = np.random.default_rng(D + taps)
    xs = [hidden(rng, n, width, dtype) for n in (70, 29)]
    want = [plain.gated_delta_rule(x64, w, mx, eps) for _, x64 in xs]
    hs = PartHarness(part.cache_specs(), dtype, max_slots=3)
    s0, s1 = hs.cache.alloc_slot(), hs.cache.alloc_slot()
    ctx = hs.step([(s0, 2), (s1, 9)])
    first = part.forward(torch.cat([xs[0][0][:2], xs[1][0][:9]]).contiguous(), ctx, views_of(hs, ctx, 2)).float().cpu().numpy()
    hs.done()
    got0 = np.concatenate([first[:2], feed(part, hs, s0, xs[0][0][2:], (1, 1, 2, 3, 1, 20, 1, 39), n_entries=2)])
    got1 = np.concatenate([first[2:], feed(part, hs, s1, xs[1][0][9:], (2, 1, 1, 16), n_entries=2)])
    close(got0, want[0], dtype, "gated delta rule, first sequence")
    close(got1, want[1], dtype, "gated delta rule, second sequence")
    hs.cache.free_slot(s0)
    s2 = hs.cache.alloc_slot()
    assert s2 == s0
    close(feed(part, hs, s2, xs[1][0], (29,), n_entries=2), want[1], dtype, "gated delta rule, a slot used again")


# ---------------------------------------------------------------------------------------------------------------
# attention with a sink and a gate per head
# ---------------------------------------------------------------------------------------------------------------
def left_part(dtype, width, H, G, D, V, scale, base, dims, eps, max_positions=1024):
    from alpacca_b200.parts import MapsAttention, RotaryEncoding
    opts = opts_of(dtype, max_positions)
    pos = RotaryEncoding(opts, D, dims, base, "neox") if dims else None
    part = MapsAttention(opts, width, H, G, D, V, pos, "m", scale, eps, qk_norm=True, sink=True, head_gate="g",
                         out_dtype=torch.float32)
    return part, {"heads": H, "kv_heads": G, "dim": D, "vdim": V, "scale": scale, "rot": {"base": base, "dims": dims}}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,D,V,dims", [(4, 2, 16, 24, 8), (6, 1, 32, 16, 32), (3, 3, 20, 12, 0), (8, 2, 64, 64, 32), (2, 2, 128, 48, 64),
                                          (4, 2, 128, 128, 64)])
def test_gated_attention(dtype, H, G, D, V, dims):
    """In portions down to one token, and whole (head sizes 64 and 128 with values of the same size then run on the
    tcgen05 kernel in bfloat16, the sink in its last step)."""
    width, eps = 40, 1e-5
    part, mx = left_part(dtype, width, H, G, D, V, 0.3, 1e4, dims, eps)
    w = short(load_part(part, seed=H + D, dtype=dtype, std=0.3), "m")
    assert {"q.norm", "k.norm", "sink", "g"} <= set(w)
    rng = np.random.default_rng(D)
    x, x64 = hidden(rng, 150, width, dtype)
    want = plain.gated_attention(x64, w, mx, eps)
    hs = PartHarness([part.cache_spec()], dtype)
    s = hs.cache.alloc_slot()
    close(feed(part, hs, s, x, (61, 2, 1, 3, 63, 1, 19)), want, dtype, "attention with a sink and a gate per head")
    close(feed(part, hs, hs.cache.alloc_slot(), x, (150,)), want, dtype, "the same, whole")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("back", [600, 64, 65, 1, 0])
@pytest.mark.parametrize("decode", [False, True])
def test_gated_attention_finds_a_planted_key(dtype, back, decode):
    """Among 700 keys one is made to point along the last token's query in one head (so that it outweighs all
    others), `back` tokens before it: far away, on the last place of a page and the first of the next, next to the
    asking token, and the asking token itself.  The plain implementation and the kernels agree, and the answer
    differs from the one without that key."""
    width, eps, T = 64, 1e-6, 700
    part, mx = left_part(dtype, width, 4, 2, 32, 16, 1.0, 1e4, 0, eps)
    w = short(load_part(part, seed=9, dtype=dtype, std=0.3), "m")
    rng = np.random.default_rng(back)
    x64 = rng.normal(0.0, 1.0, (T, width))
    at = T - 1 - back
    q_last = (w["q"] @ x64[-1]).reshape(4, 32)[1]
    x64[at] = 3.0 * np.linalg.pinv(w["k"].reshape(2, 32, width)[0]) @ q_last + (x64[-1] if back == 0 else 0.0)
    x, x64 = as_input(x64, dtype)
    want = plain.gated_attention(x64, w, mx, eps)
    if back:
        without = x64.copy()
        without[at] = rng.normal(0.0, 1.0, width)
        assert np.abs(plain.gated_attention(without, w, mx, eps)[-1] - want[-1]).max() > 0.2 * want.std()
    hs = PartHarness([part.cache_spec()], dtype, max_tokens=64 * 14)
    s = hs.cache.alloc_slot()
    got = feed(part, hs, s, x, (T - 3, 1, 1, 1) if decode else (T,))
    close(got[-3:], want[-3:], dtype, f"a planted key {back} tokens back")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("level", [-40.0, 0.5, 40.0])
def test_gated_attention_sink(dtype, level):
    """A sink far below the scores changes nothing, one far above them takes all the weight (the output is zero);
    one among the scores takes its share."""
    width, eps = 40, 1e-5
    part, mx = left_part(dtype, width, 4, 2, 16, 24, 0.3, 1e4, 8, eps)
    w = short(load_part(part, seed=3, dtype=dtype, std=0.3), "m")
    part.sink.fill_(level)
    w["sink"] = np.full(4, level)
    x, x64 = hidden(np.random.default_rng(1), 90, width, dtype)
    want = plain.gated_attention(x64, w, mx, eps)
    hs = PartHarness([part.cache_spec()], dtype)
    got = feed(part, hs, hs.cache.alloc_slot(), x, (70, 1, 1, 18))
    if level > 10:
        assert np.abs(got).max() < 1e-6 and np.abs(want).max() < 1e-6
    else:
        close(got, want, dtype, f"sink at {level}")


# ---------------------------------------------------------------------------------------------------------------
# latent attention with a window
# ---------------------------------------------------------------------------------------------------------------
def latent_part(dtype, width, H, D, R, V, Q, C, scale, base, window, eps, keep=None, own=True, prefix="m"):
    from alpacca_b200.parts import LatentAttention, RotaryEncoding
    opts = opts_of(dtype)
    part = LatentAttention(opts, width, H, D, R, V, Q, C, scale, eps, RotaryEncoding(opts, R, R, base, "llama"), prefix,
                           sink=False, window=window, keep_window=keep, head_gate="g", own_kv=own, out_dtype=torch.float32)
    mx = {"heads": H, "dim": D, "rot_dim": R, "vdim": V, "q_rank": Q, "kv_rank": C, "scale": scale,
          "rot": {"base": base, "dims": R}}
    if window:
        mx["mask"] = {"size": window}
    return part, mx


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,D,R,V,Q,C,window", [(3, 16, 8, 12, 24, 20, 70), (4, 24, 4, 16, 20, 28, 5), (2, 32, 16, 32, 24, 48, None),
                                                (5, 64, 16, 48, 80, 48, 100), (5, 12, 4, 8, 16, 12, 64), (1, 8, 2, 40, 8, 30, 65)])
def test_latent_attention_with_a_window(dtype, H, D, R, V, Q, C, window):
    width, eps = 40, 1e-5
    part, mx = latent_part(dtype, width, H, D, R, V, Q, C, 0.4, 100.0, window, eps)
    w = short(load_part(part, seed=H + D, dtype=dtype, std=0.3), "m")
    assert "sink" not in w and w["g"].shape == (H, width)
    x, x64 = hidden(np.random.default_rng(D), 200, width, dtype)
    want = plain.latent_attention(x64, w, mx, eps, plain.latent_keys(x64, w, mx, eps))
    hs = PartHarness([part.cache_spec()], dtype)
    s = hs.cache.alloc_slot()
    close(feed(part, hs, s, x, (61, 2, 1, 3, 63, 1, 19) + (1,) * 50), want, dtype, "latent attention with a window")
    hs.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [5, 64, 65, 130])
@pytest.mark.parametrize("decode", [False, True])
def test_latent_window_edges_with_a_planted_key(dtype, window, decode):
    """One key is made so that one head of the tokens after it asks for it above all others.  The token `window - 1`
    places after it still sees it, the next one does not: both rows are held to the plain implementation, and the two
    rows of the plain implementation differ, in a prompt and when the tokens are decoded one by one."""
    width, eps, T = 48, 1e-6, 330
    H, D, R, V, Q, C = 2, 16, 4, 16, 24, 28
    part, mx = latent_part(dtype, width, H, D, R, V, Q, C, 2.0, 100.0, window, eps)
    w = short(load_part(part, seed=window, dtype=dtype, std=0.3), "m")
    rng = np.random.default_rng(window)
    x64 = rng.normal(0.0, 1.0, (T, width))
    at = 190
    ask = rng.normal(0.0, 1.0, width)
    x64[at + 1:at + window + 3] = ask + 0.05 * rng.normal(0.0, 1.0, (window + 2, width))      # they all ask alike
    cq = plain.rms(w["dq"] @ ask, eps) * w["dq.norm"]
    q_un = (w["uq"] @ cq).reshape(H, D + R)[0, :D]
    c_want = w["uk"].reshape(H, D, C)[0].T @ q_un                   # the latent whose key points along that query
    x64[at] = 5.0 * np.linalg.pinv(w["dkv"][:C]) @ (c_want / w["dkv.norm"])
    x, x64 = as_input(x64, dtype)
    want = plain.latent_attention(x64, w, mx, eps, plain.latent_keys(x64, w, mx, eps))
    inside, outside = at + window - 1, at + window
    assert np.abs(want[inside] - want[outside]).max() > 0.3 * want.std()
    hs = PartHarness([part.cache_spec()], dtype, max_tokens=64 * 8)
    s = hs.cache.alloc_slot()
    cuts = (at + 2,) + (1,) * (T - at - 2) if decode else (T,)
    got = feed(part, hs, s, x, cuts)
    # a softmax this sharp passes the rounding of bfloat16 scores on at full size: more room for single numbers there
    close(got[at:at + window + 3], want[at:at + window + 3], dtype, f"the edge of a window of {window}",
          tol=(0.3, 0.03) if dtype == "bfloat16" else None)
    hs.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("own_window,reader_window", [(5, 130), (100, 7), (64, None), (None, 64)])
def test_a_layer_reads_another_layers_latent_rows(dtype, own_window, reader_window):
    """The second layer has no down-projection for keys: it reads what the first has cached, with up-projections,
    queries, gate and window of its own; the cache keeps what the wider of the two windows needs."""
    width, eps = 40, 1e-5
    wide = None if own_window is None or reader_window is None else max(own_window, reader_window)
    keep = "all" if wide is None else wide
    owner, mo = latent_part(dtype, width, 3, 16, 4, 12, 24, 28, 0.5, 50.0, own_window, eps, keep=keep, prefix="a")
    reader, mr = latent_part(dtype, width, 2, 8, 4, 20, 12, 28, 0.8, 50.0, reader_window, eps, keep=keep, own=False, prefix="b")
    assert owner.cache_spec() == reader.cache_spec() and owner.cache_spec().window == wide
    wo = short(load_part(owner, seed=1, dtype=dtype, std=0.3), "a")
    wr = short(load_part(reader, seed=2, dtype=dtype, std=0.3), "b")
    assert "dkv" not in wr and "dkv.norm" not in wr
    x, x64 = hidden(np.random.default_rng(7), 220, width, dtype)
    y, y64 = hidden(np.random.default_rng(8), 220, width, dtype)      # the second layer's own input
    kept = plain.latent_keys(x64, wo, mo, eps)
    want_o = plain.latent_attention(x64, wo, mo, eps, kept)
    want_r = plain.latent_attention(y64, wr, mr, eps, kept)
    hs = PartHarness([owner.cache_spec()], dtype, max_tokens=64 * 6)
    s = hs.cache.alloc_slot()
    got_o, got_r, at = [], [], 0
    for n in (70, 1, 1, 60, 3) + (1,) * 85:
        ctx = hs.step([(s, n)])
        view = views_of(hs, ctx, 1)
        got_o.append(owner.forward(x[at:at + n].contiguous(), ctx, view).float().cpu().numpy())
        got_r.append(reader.forward(y[at:at + n].contiguous(), ctx, view, write_cache=False).float().cpu().numpy())
        hs.done()
        at += n
    close(np.concatenate(got_o), want_o, dtype, "the layer that caches")
    close(np.concatenate(got_r), want_r, dtype, "the layer that reads")
    hs.cache.check()


# ---------------------------------------------------------------------------------------------------------------
# the router, and the experts behind it
# ---------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("E,count,keep,top", [(1, 1, 1, 1), (6, 3, 2, 2), (15, 3, 2, 5), (8, 8, 3, 3), (64, 4, 1, 9), (20, 5, 5, 7),
                                              (9, 1, 1, 9), (33, 3, 2, 20), (256, 8, 4, 8)])
def test_router(E, count, keep, top):
    """Sigmoid scores; a correction of the order of the scores, for some experts far below zero; groups scored by their
    two best members; weights without the correction and without renormalisation.  Compared where no choice is a
    close call."""
    from alpacca_b200 import ops
    rng = np.random.default_rng(E + top)
    T, width = 300, 24
    h, h64 = hidden(rng, T, width, "float32")
    router = torch.from_numpy(rng.normal(0.0, 0.6, (E, width)).astype(np.float32)).cuda()
    corr = rng.normal(-1.2, 0.8, E).astype(np.float32)
    corr[::3] -= 2.0
    w = {"router": router.double().cpu().numpy(), "correction": corr.astype(np.float64)}
    chosen, wts, margin = plain.route(h64, w, {"experts": E, "top": top, "groups": {"count": count, "keep": keep}})
    idx, got_w = ops.moe_route(h, router, T, count, keep, top, 1.0, score="sigmoid", correction=torch.from_numpy(corr).cuda(),
                               group_top=2, renorm=False)
    idx, got_w = idx.cpu().numpy(), got_w.cpu().numpy()
    sure = margin > 1e-5
    assert sure.mean() > 0.9
    assert (idx[sure] == chosen[sure]).all()
    assert np.abs(got_w[sure] - wts[sure]).max() < 1e-5
    if E >= 6 and 2 * top >= keep * (E // count):        # then some of the chosen scores ARE negative
        assert ((w["correction"][chosen[sure]] + wts[sure]) < 0).any()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T", [5, 70])
def test_routed_experts(dtype, T):
    from alpacca_b200.parts import RoutedExperts
    from types import SimpleNamespace
    width, ff, E = 40, 20, 6
    part = RoutedExperts(opts_of(dtype), width, ff, E, 2, 3, 2, 1.0, "f", activation="silu", gate_name="e{}.gate",
                         score="sigmoid", correction="correction", group_top=2, renorm=False)
    w = short(load_part(part, seed=4, dtype=dtype, std=0.3), "f")
    decided = (np.arange(E)[::-1] * 3.0 - 4.0).astype(np.float32)
    part.correction.copy_(torch.from_numpy(decided).cuda())
    w["correction"] = decided.astype(np.float64)
    x, x64 = hidden(np.random.default_rng(T), T, width, dtype)
    want = plain.experts(x64, w, {"expert": {"ff": ff}, "router": {"experts": E, "top": 2, "groups": {"count": 3, "keep": 2}}})
    got = part.forward(x, SimpleNamespace(n_tokens=T)).float().cpu().numpy()
    close(got, want, dtype, "routed experts")
