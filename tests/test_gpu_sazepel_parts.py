"""Each mechanism of the Sazepel decoder alone, against its function in tests/plain_sazepel.py: the retention
(rotated q and k, a scaled key, a norm per head, a SiLU gate), the attention whose softmax weights are mixed
across heads (norms of q, k and v without weights, a sigmoid gate), the two side by side under a block with norms
before and after every sub-layer, the routed gated experts whose router has a bias, and the normed embedding.
Sizes differ from test to test; inputs are made so that faults show."""
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_sazepel as plain
from helpers import PartHarness, load_part

pytestmark = pytest.mark.gpu

TOL = {"float32": (2e-4, 2e-5), "bfloat16": (0.12, 0.02)}      # (largest, mean) |difference| as shares of the spread
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


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


def short(weights, prefix):
    return {k[len(prefix) + 1:]: v for k, v in weights.items() if k.startswith(prefix + ".")}


def feed(part, hs, slot, x, cuts, entry=0):
    """Runs `x` through a mixer in portions; returns the outputs as one array."""
    out, at = [], 0
    for n in cuts:
        ctx = hs.step([(slot, n)])
        view = hs.cache.entry_view(entry, ctx.block_tables)
        out.append(part.forward(x[at:at + n].contiguous(), ctx, view).float().cpu().numpy())
        hs.done()
        at += n
    assert at == x.shape[0]
    return np.concatenate(out)


# ---------------------------------------------------------------------------------------------------------------
# retention
# ---------------------------------------------------------------------------------------------------------------
def retention_part(dtype, width, H, D, V, decay, base, dims, eps, max_positions=1024):
    from alpacca_b200.parts import DecayLinearAttention, RotaryEncoding
    opts = opts_of(dtype, max_positions)
    pos = RotaryEncoding(opts, D, dims, base, "neox") if dims else None
    part = DecayLinearAttention(opts, width, H, D, V, decay, eps, "m", activation=None, position=pos,
                                key_scale=float(D) ** -0.5, head_norm=True, norm_weight=False, gate="silu",
                                out_dtype=torch.float32)
    mx = {"heads": H, "dim": D, "vdim": V, "decay": list(decay), "rot": {"base": base, "dims": dims}}
    return part, mx


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,D,V,decay,base,dims", [
    (2, 16, 24, (0.7, 1.0), 100.0, 16), (1, 24, 40, (0.99,), 1e4, 12), (3, 64, 20, (0.3, 0.9, 0.999), 1e6, 64),
    (2, 128, 36, (0.95, 0.5), 50.0, 2), (1, 40, 70, (0.9,), 10.0, 0), (1, 6, 33, (0.8,), 500.0, 4),
    (5, 32, 32, (0.984375, 0.99, 0.995, 0.999, 1.0), 1e6, 32), (1, 200, 130, (0.97,), 1e3, 100)])
def test_retention(dtype, H, D, V, decay, base, dims):
    """Two sequences side by side, fed in portions of unequal sizes down to one token; the state is carried from
    step to step and the rotation goes on at the right position.  Rotations over all, part and none of a vector."""
    width, eps = 56, 1e-5
    part, mx = retention_part(dtype, width, H, D, V, decay, base, dims, eps)
    w = short(load_part(part, seed=H * 100 + D, dtype=dtype, std=0.25), "m")
    assert set(w) == {"q", "k", "v", "g", "o"}
    rng = np.random.default_rng(D)
    lens = (75, 31)
    xs = [hidden(rng, n, width, dtype) for n in lens]
    want = [plain.retention(x64, w, mx, eps)[0] for _, x64 in xs]
    hs = PartHarness([part.cache_spec()], dtype, max_slots=3)
    s0, s1 = hs.cache.alloc_slot(), hs.cache.alloc_slot()
    ctx = hs.step([(s0, 20), (s1, 9)])
    view = hs.cache.entry_view(0, ctx.block_tables)
    first = part.forward(torch.cat([xs[0][0][:20], xs[1][0][:9]]).contiguous(), ctx, view).float().cpu().numpy()
    hs.done()
    got0 = np.concatenate([first[:20], feed(part, hs, s0, xs[0][0][20:], (1, 2, 17, 1, 34))])
    got1 = np.concatenate([first[20:], feed(part, hs, s1, xs[1][0][9:], (2, 2, 1, 17))])
    close(got0, want[0], dtype, "retention, first sequence")
    close(got1, want[1], dtype, "retention, second sequence")
    # the state of a slot that is given back and taken again starts at zero
    hs.cache.free_slot(s0)
    s2 = hs.cache.alloc_slot()
    assert s2 == s0
    close(feed(part, hs, s2, xs[1][0], (31,)), want[1], dtype, "retention, a slot used again")
    state = hs.cache.entry_view(0, None).state[s2].double().cpu().numpy()
    close(state, plain.retention(xs[1][1], w, mx, eps)[1], dtype, "retention, the state",
          tol=(0.05, 0.01) if dtype == "bfloat16" else None)
    # a long prompt in one step is cut into pieces that are walked side by side; the next portion starts from the
    # state that they leave, at the position where they end
    long_x, long64 = hidden(rng, 330, width, dtype)
    s3 = hs.cache.alloc_slot()
    close(feed(part, hs, s3, long_x, (300, 28, 2)), plain.retention(long64, w, mx, eps)[0], dtype,
          "retention, a long prompt in pieces")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("decode", [False, True])
def test_retention_keeps_a_far_token_and_forgets_by_its_decay(dtype, decode):
    """One early token carries a value that no other has; nine hundred tokens later a query asks for its key.  The
    head that does not decay returns the value at full size, the head with decay a returns a^distance of it, and the
    head norm then shows only the direction: the plain implementation and the kernel agree, and the answer differs
    from the one without the early token."""
    width, eps, H, D, V = 40, 1e-6, 2, 16, 24
    part, mx = retention_part(dtype, width, H, D, V, (1.0, 0.99), 1e4, 0, eps, max_positions=2048)
    w = short(load_part(part, seed=5, dtype=dtype, std=0.02), "m")
    Wt = part.proj.weight.float()
    # column 0 drives the last dim of every query, column 2 that of every key, column 1 value column 1 of every head
    for name, off, size in (("q", part.offsets[0], D), ("k", part.offsets[1], D), ("v", part.offsets[2], V)):
        w[name][:, :3] = 0.0
        Wt[off:off + H * size, :3] = 0.0
    for a in range(H):
        w["q"][a * D + D - 1, 0] = Wt[part.offsets[0] + a * D + D - 1, 0] = 4.0
        w["k"][a * D + D - 1, 2] = Wt[part.offsets[1] + a * D + D - 1, 2] = 4.0
        w["v"][a * V + 1, 1] = Wt[part.offsets[2] + a * V + 1, 1] = 2.0
    part.proj.weight = Wt.to(part.proj.weight.dtype).contiguous()
    n, planted, asks = 960, 7, 950
    rng = np.random.default_rng(9)
    x, x64 = hidden(rng, n, width, dtype)
    x[:, :3] = 0.0
    x64[:, :3] = 0.0
    for p, col in ((planted, 2), (planted, 1), (asks, 0)):
        x[p, col] = x64[p, col] = 3.0
    want = plain.retention(x64, w, mx, eps)[0]
    x_without = x64.copy()
    x_without[planted, 1:3] = 0.0
    assert np.abs(want[asks] - plain.retention(x_without, w, mx, eps)[0][asks]).max() > 0.2 * np.abs(want).max()
    hs = PartHarness([part.cache_spec()], dtype, max_tokens=2048, max_slots=2, max_positions=2048)
    s = hs.cache.alloc_slot()
    cuts = (900,) + (1,) * 60 if decode else (n,)
    got = feed(part, hs, s, x, cuts)
    close(got, want, dtype, "retention with a planted token")
    close(got[asks], want[asks], dtype, "retention, the token that asks", tol=(0.05, 0.02) if dtype == "bfloat16" else (1e-3, 2e-4))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_retention_rotation_depends_on_the_distance_alone(dtype):
    """With all of q and k rotated and no decay, q_t . k_s depends on t - s only: the same tokens fed from position
    0 and from position 600 (after a prefix whose keys and values are zero) give the same outputs."""
    width, eps, H, D, V = 32, 1e-5, 2, 32, 16
    part, mx = retention_part(dtype, width, H, D, V, (1.0, 1.0), 1e4, 32, eps, max_positions=2048)
    w = short(load_part(part, seed=6, dtype=dtype, std=0.25), "m")
    rng = np.random.default_rng(1)
    x, x64 = hidden(rng, 50, width, dtype)
    hs = PartHarness([part.cache_spec()], dtype, max_tokens=2048, max_slots=2, max_positions=2048)
    s = hs.cache.alloc_slot()
    at0 = feed(part, hs, s, x, (50,))
    s2 = hs.cache.alloc_slot()
    zeros = torch.zeros((600, width), dtype=x.dtype, device="cuda")
    feed(part, hs, s2, zeros, (600,))
    at600 = feed(part, hs, s2, x, (30,) + (1,) * 20)
    want = plain.retention(x64, w, mx, eps)[0]
    close(at0, want, dtype, "retention at position 0")
    close(at600, want, dtype, "retention at position 600", tol=(0.12, 0.02) if dtype == "bfloat16" else (2e-3, 2e-4))


# ---------------------------------------------------------------------------------------------------------------
# attention whose softmax weights are mixed across heads
# ---------------------------------------------------------------------------------------------------------------
def mixed_attention_part(dtype, width, H, G, D, V, scale, eps, seed, std=0.3, max_positions=1024):
    from alpacca_b200.parts import MapsAttention
    part = MapsAttention(opts_of(dtype, max_positions), width, H, G, D, V, None, "a", scale, eps, qk_norm=True,
                         qk_norm_weight=False, value_norm=True, head_mix="talk", gate="g", out_dtype=torch.float32)
    w = short(load_part(part, seed=seed, dtype=dtype, std=std), "a")
    assert set(w) == {"q", "k", "v", "g", "o", "talk"}
    # a mixing matrix with entries of both signs and of order 1, far from the identity
    talk = np.random.default_rng(seed).normal(0.0, 0.7, (H, H)) + 0.5 * np.eye(H)
    part.talk.copy_(torch.from_numpy(talk).float())
    w["talk"] = part.talk.double().cpu().numpy()
    mx = {"heads": H, "kv_heads": G, "dim": D, "vdim": V, "scale": scale}
    return part, w, mx


MIXED_SHAPES = [
    # H, G, D, V: groups of 2; one key/value head for all; as many as heads; a single head; sizes that take the
    # tensor-core tiles in bfloat16 (steps of 16, the values of all heads within 256) and ones that do not
    (4, 2, 16, 24), (8, 1, 32, 16), (3, 3, 20, 12), (1, 1, 24, 40), (6, 2, 48, 48), (8, 4, 64, 64), (2, 2, 72, 136),
    (6, 3, 16, 80), (4, 4, 128, 32),
    # the values of all heads are more than 256 numbers: the tile kernel takes them 256 columns at a time
    (8, 4, 32, 80), (4, 4, 16, 128), (3, 3, 48, 176),
]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,D,V", MIXED_SHAPES)
def test_mixed_attention_whole_portions_and_single_tokens(dtype, H, G, D, V):
    """A sequence of 150 tokens: whole; in portions down to two tokens; its last 90 tokens one by one across the
    page borders at 64 and 128; beside another sequence in the same step, and both going on by a token."""
    width, eps = 40, 1e-5
    part, w, mx = mixed_attention_part(dtype, width, H, G, D, V, 3.0, eps, seed=H * 10 + D)
    rng = np.random.default_rng(D + V)
    x, x64 = hidden(rng, 150, width, dtype)
    y, y64 = hidden(rng, 40, width, dtype)
    want, want_y = plain.talking_attention(x64, w, mx, eps), plain.talking_attention(y64, w, mx, eps)
    hs = PartHarness([part.cache_spec()], dtype, max_slots=4)
    # bfloat16: a mixing matrix with entries of order 1 and both signs over up to 8 heads adds the heads' roundings up
    # (largest seen 0.18 of the spread for one number, 0.010 for the mean)
    tol = (0.3, 0.03) if dtype == "bfloat16" else None
    for cuts in ((150,), (2, 3, 59, 1, 64, 2, 19), (20, 130), (60,) + (1,) * 90, (2,) * 75):
        s = hs.cache.alloc_slot()
        close(feed(part, hs, s, x, cuts), want, dtype, f"mixed attention in portions {cuts[:4]}", tol=tol)
        hs.cache.free_slot(s)
    s, s2 = hs.cache.alloc_slot(), hs.cache.alloc_slot()
    ctx = hs.step([(s2, 40), (s, 100)])
    view = hs.cache.entry_view(0, ctx.block_tables)
    both = part.forward(torch.cat([y, x[:100]]).contiguous(), ctx, view).float().cpu().numpy()
    hs.done()
    close(both[:40], want_y, dtype, "mixed attention, the short sequence of a batch", tol=tol)
    close(both[40:], want[:100], dtype, "mixed attention, the long sequence of a batch", tol=tol)
    ctx = hs.step([(s2, 1), (s, 1)])
    view = hs.cache.entry_view(0, ctx.block_tables)
    y2, y2_64 = hidden(rng, 1, width, dtype)
    nxt = part.forward(torch.cat([y2, x[100:101]]).contiguous(), ctx, view).float().cpu().numpy()
    hs.done()
    one_row = (0.3, 0.06) if dtype == "bfloat16" else None      # the mean over one row's few numbers
    close(nxt[1:], want[100:101], dtype, "mixed attention, a decode step of two sequences", tol=one_row)
    close(nxt[:1], plain.talking_attention(np.concatenate([y64, y2_64]), w, mx, eps)[40:], dtype,
          "mixed attention, the other row", tol=one_row)
    hs.cache.check()


@pytest.mark.parametrize("group,most", [(128, 512), (128, 256), (64, 512), (256, 256), (48, 96)])
@pytest.mark.parametrize("H,G,D,V", [(8, 4, 32, 80), (4, 4, 16, 128), (3, 3, 48, 176), (2, 2, 144, 96), (4, 1, 64, 32)])
def test_mixed_attention_wide_value_rows_in_groups_of_warps(H, G, D, V, group, most, monkeypatch):
    """The tile kernel takes a token's value row in launches of up to `most` columns, and within a launch 1, 2 or 4
    groups of warps take `group` columns each: every split gives the same attention (bfloat16)."""
    from alpacca_b200 import ops
    monkeypatch.setattr(ops, "TALK_GROUP_COLUMNS", group)
    monkeypatch.setattr(ops, "TALK_TILE_COLUMNS", most)
    width, eps = 40, 1e-5
    part, w, mx = mixed_attention_part("bfloat16", width, H, G, D, V, 3.0, eps, seed=H + V)
    x, x64 = hidden(np.random.default_rng(D), 150, width, "bfloat16")
    want = plain.talking_attention(x64, w, mx, eps)
    hs = PartHarness([part.cache_spec()], "bfloat16", max_slots=2)
    for cuts in ((150,), (70, 3, 77)):
        s = hs.cache.alloc_slot()
        close(feed(part, hs, s, x, cuts), want, "bfloat16", f"mixed attention, {group} of {most} columns", tol=(0.3, 0.03))
        hs.cache.free_slot(s)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,D,V", [(4, 2, 16, 24), (4, 2, 32, 32), (2, 1, 20, 12)])
@pytest.mark.parametrize("decode", [False, True, "few parts"])
@pytest.mark.parametrize("planted", [5, 63, 64, 620, 621])
def test_mixed_attention_finds_a_key_far_back(dtype, H, G, D, V, decode, planted, monkeypatch):
    """One token carries a key and a value that no other has; token 620 (on the tenth page) has queries that ask for
    that key, with a scale that lets it outweigh the hundreds of others.  Only ONE head's queries ask; the mixing
    matrix spreads that head's weights to the others, each of which reads the planted value from its own key/value
    head.  The key is planted far back (token 5), on the last place of the first page and the first of the second,
    on the asking token itself (a token sees its own key) and on the one after it (which it must not see).  In
    decoding the ten pages of keys are taken one page per CTA, or ("few parts") in runs of several pages per CTA."""
    from alpacca_b200 import ops
    if decode == "few parts":
        monkeypatch.setattr(ops, "TALK_DECODE_BLOCKS", 3 * G)
    width, eps, scale = 40, 1e-6, 12.0
    part, w, mx = mixed_attention_part(dtype, width, H, G, D, V, scale, eps, seed=D, std=0.05, max_positions=1024)
    Wt = part.qkv.weight.float()
    n_q, n_k = H * D, G * D
    per = H // G
    for name in ("q", "k", "v"):
        w[name][:, :3] = 0.0
    Wt[:n_q + n_k + G * V, :3] = 0.0
    asking = H - 1                                # head H-1 asks; the package keeps query vector j*G + c for head c*per + j
    row = ((asking % per) * G + asking // per) * D + D - 1
    w["q"][asking * D + D - 1, 0] = Wt[row, 0] = 30.0
    for g in range(G):
        w["k"][g * D + D - 1, 2] = Wt[n_q + g * D + D - 1, 2] = 30.0
        w["v"][g * V + 1 + g, 1] = Wt[n_q + n_k + g * V + 1 + g, 1] = 30.0      # another column in every value head
    part.qkv.weight = Wt.to(part.qkv.weight.dtype).contiguous()
    n, asks = 640, 620
    rng = np.random.default_rng(V)
    x, x64 = hidden(rng, n, width, dtype)
    x[:, :3] = 0.0
    x64[:, :3] = 0.0
    for p, col in ((planted, 2), (planted, 1), (asks, 0)):
        x[p, col] = x64[p, col] = 3.0
    want = plain.talking_attention(x64, w, mx, eps)
    x_without = x64.copy()
    x_without[planted, 1:3] = 0.0
    gap = np.abs(want[asks] - plain.talking_attention(x_without, w, mx, eps)[asks]).max()
    if planted <= asks:
        assert gap > 0.3 * np.abs(want[asks]).max(), "the planted key does not show in the plain implementation"
    else:
        assert gap == 0.0, "a later token's key shows in the plain implementation"
    hs = PartHarness([part.cache_spec()], dtype, max_slots=2)
    s = hs.cache.alloc_slot()
    cuts = (600,) + (1,) * 40 if decode else (n,)
    got = feed(part, hs, s, x, cuts)
    # (bfloat16: the spread of the outputs is small beside the planted value, whose rounding is what differs)
    close(got, want, dtype, "mixed attention with a planted key", tol=(0.5, 0.03) if dtype == "bfloat16" else None)
    close(got[asks], want[asks], dtype, "mixed attention, the token that asks",
          tol=(0.06, 0.02) if dtype == "bfloat16" else (1e-3, 2e-4))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_attention_values_are_cached_normed_and_side_by_side(dtype):
    from alpacca_b200.parts import KVSpec
    width, eps, H, G, D, V = 40, 1e-3, 4, 2, 16, 24
    part, w, mx = mixed_attention_part(dtype, width, H, G, D, V, 1.0, eps, seed=1)
    assert part.cache_spec() == KVSpec(G, D, None, value_heads=1, value_dim=G * V)
    x, x64 = hidden(np.random.default_rng(0), 70, width, dtype)
    x[3] *= 2.0 ** -7                   # a token whose vectors are small against eps: eps is inside the root
    x64 = x.double().cpu().numpy()
    hs = PartHarness([part.cache_spec()], dtype, max_slots=1)
    s = hs.cache.alloc_slot()
    close(feed(part, hs, s, x[:66], (66,)), plain.talking_attention(x64, w, mx, eps)[:66], dtype, "mixed attention, eps")
    ctx = hs.step([(s, 4)])
    view = hs.cache.entry_view(0, ctx.block_tables)
    part.forward(x[66:].contiguous(), ctx, view)
    hs.done()
    tab = view.block_table[0].cpu().numpy()
    v = plain.unit((x64 @ w["v"].T).reshape(70, G, V), eps).reshape(70, G * V)
    k = plain.unit((x64 @ w["k"].T).reshape(70, G, D), eps)
    got_v = torch.cat([view.v[int(tab[0]), 0], view.v[int(tab[1]), 0, :6]]).double().cpu().numpy()
    got_k = torch.cat([view.k[int(tab[0])], view.k[int(tab[1]), :, :6]], dim=1).double().cpu().numpy()
    close(got_v, v, dtype, "cached values", tol=(0.02, 0.005) if dtype == "bfloat16" else None)
    close(got_k.transpose(1, 0, 2), k, dtype, "cached keys", tol=(0.02, 0.005) if dtype == "bfloat16" else None)


# ---------------------------------------------------------------------------------------------------------------
# the kernel after a sub-layer; two mixers side by side; the block
# ---------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("E,T", [(40, 1), (37, 5), (256, 33), (1000, 3), (4096, 2)])
@pytest.mark.parametrize("two", [False, True])
@pytest.mark.parametrize("then", [False, True])
def test_norm_of_a_sublayer_output_added_to_the_stream(dtype, E, T, two, then):
    from alpacca_b200 import ops
    rng = np.random.default_rng(E + T)
    eps = 1e-5
    res = torch.from_numpy(rng.normal(0, 2.0, (T, E)).astype(np.float32)).cuda()
    a, a64 = hidden(rng, T, E, dtype)
    b, b64 = hidden(rng, T, E, dtype)
    b64 = b64 * 8.0                     # the two outputs differ in size: each is normed before the sum
    b = (b.float() * 8.0).to(b.dtype)
    wts = [torch.from_numpy(rng.normal(1.0, 0.5, E).astype(np.float32)).cuda() for _ in range(4)]
    w, wa, wb, wn = (t.double().cpu().numpy() for t in wts)
    r64 = res.double().cpu().numpy()
    y = 0.5 * (plain.unit(a64, eps) * wa + plain.unit(b64, eps) * wb) if two else a64
    want = r64 + plain.unit(y, eps) * w
    out = torch.empty((T, E), dtype=DT[dtype], device="cuda") if then else None
    more = {"b": b, "wa": wts[1], "wb": wts[2]} if two else {}
    ops.post_norm_add(res, a, wts[0], eps, None, next_weight=wts[3] if then else None, out=out, **more)
    close(res.cpu().numpy(), want, "float32", "the stream after the sub-layer", tol=(5e-6, 5e-7))
    if then:
        close(out.float().cpu().numpy(), plain.unit(want, eps) * wn, dtype, "the next norm's output",
              tol=(0.04, 0.004) if dtype == "bfloat16" else None)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("with_ff", [True, False])
def test_block_with_two_mixers_side_by_side(dtype, with_ff):
    """x += n1b(half the sum of the two normed mixers (n1(x))); x += n2b(experts(n2(x))): a block of its own, fed in
    portions, with one cache entry for the attention's keys and values and one for the retention's state."""
    from alpacca_b200.parts import RMSNorm, RoutedExperts, SandwichBlock, SideBySide
    from alpacca_b200.parts.block import HiddenStream
    width, eps = 48, 1e-5
    opts = opts_of(dtype)
    norm = lambda n: RMSNorm(opts, width, eps, n, weight_suffix="", scalar=True)      # noqa: E731
    left, lw, lmx = mixed_attention_part(dtype, width, 4, 2, 16, 24, 2.0, eps, seed=3)
    right, rmx = retention_part(dtype, width, 3, 8, 12, (0.5, 0.9, 1.0), 100.0, 4, eps)
    mixer = SideBySide(opts, width, left, right, eps, "b.mix")
    mlp = {"kind": "moe", "expert": {"ff": 20}, "router": {"experts": 4, "top": 2}}
    ffn = RoutedExperts(opts, width, 20, 4, 2, 1, 1, 1.0, "b.mlp", activation="silu", router_bias=True,
                        gate_name="e{}.gate") if with_ff else None
    block = SandwichBlock(norm("b.norm1"), mixer, norm("b.norm1b"), *((norm("b.norm2"), ffn, norm("b.norm2b")) if with_ff else ()))
    # the two mixers were loaded by their own helpers; the rest here
    rw = short(load_part(right, seed=4, dtype=dtype, std=0.25), "m")
    w = {}
    for part in [block.norm1, block.post1] + ([block.norm2, block.post2, ffn] if with_ff else []):
        w.update(load_part(part, seed=len(w) + 5, dtype=dtype, std=0.3))
    mixer.load_own(lambda spec: torch.from_numpy(np.random.default_rng(len(spec.name)).normal(1.0, 0.4, spec.shape)
                                                 .astype(np.float32)).cuda())
    w64 = {"left.out": mixer.w_left.double().cpu().numpy(), "right.out": mixer.w_right.double().cpu().numpy()}
    w64.update({"left." + k: v for k, v in lw.items()})
    w64.update({"right." + k: v for k, v in rw.items()})
    assert len(block.cache_specs()) == 2
    rng = np.random.default_rng(8)
    x, x64 = hidden(rng, 90, width, dtype)
    x64 = x64 * 3.0
    hs = PartHarness(block.cache_specs(), dtype, max_slots=2)
    s = hs.cache.alloc_slot()
    got, at = [], 0
    for n in (50, 2, 1, 37):
        ctx = hs.step([(s, n)])
        views = [hs.cache.entry_view(e, ctx.block_tables) for e in range(2)]
        stream = HiddenStream((x[at:at + n].float() * 3.0).contiguous())
        block.forward(stream, ctx, views)
        hs.done()
        assert stream.delta is None
        got.append(stream.residual[:n].double().cpu().numpy())
        at += n
    mx = {"left": lmx, "right": rmx}
    h = plain.unit(x64, eps) * w["b.norm1"]
    want = x64 + plain.unit(plain.side_by_side(h, w64, mx, eps), eps) * w["b.norm1b"]
    if with_ff:
        h = plain.unit(want, eps) * w["b.norm2"]
        want = want + plain.unit(plain.experts(h, short(w, "b.mlp"), mlp), eps) * w["b.norm2b"]
    close(np.concatenate(got) - x64, want - x64, dtype, "block with two mixers side by side",
          tol=(0.15, 0.02) if dtype == "bfloat16" else None)


# ---------------------------------------------------------------------------------------------------------------
# routed experts, embedding
# ---------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("E,top,ff,T", [(4, 2, 20, 5), (3, 1, 16, 5), (5, 5, 24, 7), (1, 1, 12, 3), (8, 2, 96, 50),
                                        (6, 3, 8, 50), (7, 4, 36, 1), (2, 1, 40, 300)])
def test_routed_gated_experts_with_a_router_bias(dtype, E, top, ff, T):
    """Few tokens read the chosen experts' rows; many tokens in bfloat16 run all experts in two products.  The bias
    is of the order of the logits, so that a choice made without it differs."""
    from alpacca_b200.parts import RoutedExperts
    width = 48
    part = RoutedExperts(opts_of(dtype), width, ff, E, top, 1, 1, 1.0, "f", activation="silu", router_bias=True,
                         gate_name="e{}.gate")
    w = short(load_part(part, seed=E, dtype=dtype, std=0.3), "f")
    bias = np.random.default_rng(E).normal(0.0, 2.0, E).astype(np.float32)
    part.bias.copy_(torch.from_numpy(bias))
    w["router.b"] = part.bias.double().cpu().numpy()
    x, x64 = hidden(np.random.default_rng(ff), T, width, dtype)
    mlp = {"router": {"experts": E, "top": top}}
    if E > top:
        without = dict(w, **{"router.b": np.zeros(E)})
        assert (plain.route(x64, without, mlp["router"])[0] != plain.route(x64, w, mlp["router"])[0]).any() or T < 3
    margins = []
    want = plain.experts(x64, w, mlp, margins)
    out = part.forward(x, SimpleNamespace(n_tokens=T)).float().cpu().numpy()
    sure = margins[0] > 1e-3
    close(out[sure], want[sure], dtype, "routed experts")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_embedding_with_a_norm(dtype):
    from alpacca_b200.parts import RMSNorm, TokenEmbedding
    opts, eps, width, vocab = opts_of(dtype), 1e-2, 37, 50
    emb = TokenEmbedding(opts, vocab, width, "embed", weight_suffix="",
                         norm=RMSNorm(opts, width, eps, "embed.norm", weight_suffix="", scalar=True))
    w = load_part(emb, seed=2, dtype=dtype, std=0.5)
    assert w["embed.norm"].shape == ()
    tokens = torch.tensor([3, 0, 49, 3, 7], dtype=torch.int32, device="cuda")
    got = emb.forward(tokens, 5)
    assert got.dtype == torch.float32
    close(got.cpu().numpy(), plain.unit(w["embed"][[3, 0, 49, 3, 7]], eps) * w["embed.norm"], "float32", "normed embedding")
