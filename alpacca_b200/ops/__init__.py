"""Python side of the CUDA kernels: argument checks and the ctypes calls.

Every function here runs a hand-written sm_100a kernel from `csrc/` on the
current CUDA stream.  There is no CPU implementation behind them: tensors that
are not on a CUDA device are refused, and a library that cannot be built or
loaded raises.  Shapes, dtypes, strides and index ranges that a kernel relies
on are checked here, on the host, before the launch, since a kernel given a
bad pointer or size would fault the device rather than raise.
"""
from __future__ import annotations

import ctypes
import math

import torch

from . import build

_DT = {torch.float32: 0, torch.bfloat16: 1}


class KernelError(RuntimeError):
    pass


# The library products of this package (`torch.mm` on bfloat16 operands) add in float32 throughout: the
# library may not reduce partial sums of a split inner dimension in bfloat16 (measured on a B200 at the 1B
# sizes: the same step times and the same results either way; the setting makes it a rule).
torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False


def _lib(name):
    return build.load(name)


# torch's current stream of the current device as a raw handle.  The direct bindings cost a
# fraction of a microsecond; torch.cuda.current_stream() builds a Stream object each time
# (15 us, and a prefill step asks a hundred times).
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream():
    if _raw_stream is not None and _raw_device is not None:
        return ctypes.c_void_p(_raw_stream(_raw_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _p(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _need(cond, msg):
    if not cond:
        raise KernelError(msg)


def _cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("alpacca_b200 kernels run on CUDA tensors only (there is no CPU path); "
                              f"got a tensor on {t.device}")


launches = 0     # kernels of this package launched so far (the benchmark reports the count)
_timeline = None  # while `timers()` is active: [(operation, event recorded after its launch), ...]


class Timers:
    """Device time per kind of operation, for steps that are issued one launch after the other (not for
    graph replays).  An event is recorded after every launch of this package (and after the library
    products it calls); an operation's time is the time from the event before it to its own, so what
    the device idles between two launches counts for the later one.

        with ops.timers() as t:
            engine.step(entries)
        print(t.table())
    """

    def __init__(self):
        self.marks = []

    def __enter__(self):
        global _timeline
        if _timeline is not None:
            raise KernelError("ops.timers() is already active")
        torch.cuda.synchronize()
        start = torch.cuda.Event(enable_timing=True)
        start.record()
        self.marks = [("start", start)]
        _timeline = self.marks
        return self

    def __exit__(self, *exc):
        global _timeline
        _timeline = None
        torch.cuda.synchronize()
        return False

    def totals(self) -> dict:
        """{operation: (launches, microseconds)} in the order of first appearance."""
        out: dict = {}
        for (_, before), (what, after) in zip(self.marks, self.marks[1:]):
            n, us = out.get(what, (0, 0.0))
            out[what] = (n + 1, us + before.elapsed_time(after) * 1e3)
        return out

    def table(self) -> str:
        tot = self.totals()
        whole = sum(us for _, us in tot.values()) or 1.0
        lines = [f"{'operation':<24} {'launches':>8} {'us':>10} {'share':>7}"]
        for what, (n, us) in sorted(tot.items(), key=lambda kv: -kv[1][1]):
            lines.append(f"{what:<24} {n:>8} {us:>10.1f} {100 * us / whole:>6.1f}%")
        lines.append(f"{'total':<24} {sum(n for n, _ in tot.values()):>8} {whole:>10.1f}")
        return "\n".join(lines)


def timers() -> Timers:
    return Timers()


def timing() -> bool:
    """Whether `timers()` is active: every launch is followed by an event then, so nothing may be captured
    into a graph or replayed from one (a replay is opaque to the events)."""
    return _timeline is not None


def _mark(what):
    if _timeline is not None:
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        _timeline.append((what, ev))


def _check(rc, what, kernels=1):
    """`kernels`: how many kernels the entry point launched (some run two or three in a row)."""
    global launches
    launches += kernels
    _mark(what)
    if rc != 0:
        if rc >= 1000:
            raise KernelError(f"{what}: CUDA error {rc - 1000} at launch")
        raise KernelError(f"{what}: the kernel refused its arguments (code {rc})")


def _dt(t):
    code = _DT.get(t.dtype)
    if code is None:
        raise KernelError(f"dtype {t.dtype} is not supported by the kernels (float32 or bfloat16)")
    return code


def _i32(t, n=None, name="index tensor"):
    if t.dtype != torch.int32 or not t.is_contiguous():
        raise KernelError(f"{name} must be a contiguous int32 tensor")
    if n is not None and t.numel() < n:
        raise KernelError(f"{name} holds {t.numel()} entries, {n} needed")


# ---------------------------------------------------------------------------

def embed_rows(table, tokens, out):
    """out[i,:] = table[tokens[i],:] as float32.  table [V,E] f32/bf16, tokens int32 [n], out f32 [n,E]."""
    _cuda(table, tokens, out)
    n = tokens.numel()
    _i32(tokens, name="tokens")
    _need(table.dim() == 2 and table.is_contiguous(), "embedding table must be contiguous [V,E]")
    _need(out.dtype == torch.float32 and out.is_contiguous() and out.shape[-1] == table.shape[1]
          and out.numel() >= n * table.shape[1], "embed_rows: out must be float32 [n,E]")
    _check(_lib("elementwise").ab_embed_rows(_p(table), _dt(table), _p(tokens), _p(out), n,
                                             table.shape[1], table.shape[0], _stream()), "embed_rows")
    return out


def add_rmsnorm(residual, delta, weight, eps, out, rows=None, n_rows=None):
    """Fused residual add and RMSNorm.

    residual f32 [T,E] (updated in place with `delta` when `rows` is None),
    delta [T,E] of the activation dtype or None, weight f32 [E], out [n,E] of
    the activation dtype or None (add only).  `rows` (int32 [n]) picks the
    source rows and leaves the residual untouched.
    """
    _cuda(residual, delta, weight, out, rows)
    E = residual.shape[-1]
    T = residual.numel() // E
    _need(residual.dtype == torch.float32 and residual.is_contiguous(), "residual must be contiguous float32")
    _need(weight.dtype == torch.float32 and weight.numel() == E and weight.is_contiguous(),
          "norm weight must be float32 [E]")
    if delta is not None:
        _need(delta.is_contiguous() and delta.numel() == residual.numel(), "delta must match the residual")
    if rows is not None:
        n = rows.numel() if n_rows is None else n_rows
        _i32(rows, n, "rows")
    else:
        n = T if n_rows is None else n_rows
        _need(n <= T, "add_rmsnorm: more rows than the residual has")
    act = out if out is not None else delta
    _need(act is not None, "add_rmsnorm needs delta or out")
    if out is not None:
        _need(out.is_contiguous() and out.numel() >= n * E, "add_rmsnorm: out too small")
        if delta is not None:
            _need(out.dtype == delta.dtype, "add_rmsnorm: delta and out differ in dtype")
    _check(_lib("elementwise").ab_add_rmsnorm(_p(residual), _p(delta), _p(weight), _p(out), _dt(act), _p(rows),
                                              n, E, ctypes.c_float(eps), _stream()), "add_rmsnorm")
    return out


def residual_add(residual, delta, n_rows=None):
    """residual[:n] += delta[:n] in float32 (delta float32 or bfloat16, the same width)."""
    _cuda(residual, delta)
    E = residual.shape[-1]
    n = residual.numel() // E if n_rows is None else n_rows
    _need(residual.dtype == torch.float32 and residual.is_contiguous() and delta.is_contiguous()
          and delta.shape[-1] == E and residual.numel() >= n * E and delta.numel() >= n * E,
          "residual_add: residual float32 [T,E], delta [T,E]")
    _check(_lib("elementwise").ab_residual_add(_p(residual), _p(delta), _dt(delta), ctypes.c_longlong(n * E), _stream()),
           "residual_add")
    return residual


def add_bias(y, bias):
    """y[t,j] += bias[j] in place; bias float32."""
    _cuda(y, bias)
    N = y.shape[-1]
    _need(y.is_contiguous() and bias.dtype == torch.float32 and bias.numel() == N and bias.is_contiguous(),
          "add_bias: y contiguous [..,N], bias float32 [N]")
    _check(_lib("elementwise").ab_add_bias(_p(y), _dt(y), _p(bias), y.numel() // N, N, _stream()), "add_bias")
    return y


def rope_append(qkv, cos, sin, tok_pos, tok_seq, block_table, k_pages, v_pages, n_tokens, H, K, D,
                n_rot, pairing, write_cache=True, max_len=None):
    """Rotates q and k of `qkv` [T,(H+2K)D] by position and appends k, v to the pages.

    cos/sin: float32 [P, n_rot/2] or None (no rotation); pairing 0 = (2i,2i+1),
    1 = (i, n_rot/2+i).  k_pages/v_pages: [n_pages, K, page, D] of qkv's dtype.
    `max_len`: the longest sequence of the step after it (tok_pos < max_len); with it the tables'
    rows and the block table's width are checked here, else the caller guarantees tok_pos < P
    and that the block table covers tok_pos.
    """
    _cuda(qkv, cos, sin, tok_pos, tok_seq, block_table, k_pages, v_pages)
    _need(qkv.is_contiguous() and qkv.shape[-1] == (H + 2 * K) * D and qkv.numel() >= n_tokens * (H + 2 * K) * D,
          "rope_append: qkv must be contiguous [T,(H+2K)*D]")
    _i32(tok_pos, n_tokens, "tok_pos")
    _i32(tok_seq, n_tokens, "tok_seq")
    _need(block_table.dtype == torch.int32 and block_table.dim() == 2 and block_table.is_contiguous(),
          "block_table must be contiguous int32 [B,W]")
    if cos is not None:
        _need(sin is not None and cos.dtype == torch.float32 and sin.dtype == torch.float32
              and cos.is_contiguous() and sin.is_contiguous() and cos.shape == sin.shape
              and cos.shape[-1] == n_rot // 2, "rope tables must be float32 [P, n_rot/2]")
        _need(max_len is None or max_len <= cos.shape[0],
              f"rope tables hold {cos.shape[0]} positions, the step reaches position {max_len}")
    page_size = k_pages.shape[2]
    _need(max_len is None or max_len <= block_table.shape[1] * page_size,
          f"the block table covers {block_table.shape[1] * page_size} positions, the step reaches {max_len}")
    if write_cache:
        _need(k_pages.dtype == qkv.dtype and v_pages.dtype == qkv.dtype and k_pages.is_contiguous()
              and v_pages.is_contiguous() and tuple(k_pages.shape[1:]) == (K, page_size, D)
              and k_pages.shape == v_pages.shape, "cache pages must be contiguous [n_pages,K,page,D] of qkv's dtype")
    _check(_lib("elementwise").ab_rope_append(
        _p(qkv), _dt(qkv), _p(cos), _p(sin), _p(tok_pos), _p(tok_seq), _p(block_table), block_table.shape[1],
        _p(k_pages), _p(v_pages), n_tokens, H, K, D, n_rot, pairing, page_size, 1 if write_cache else 0,
        _stream()), "rope_append")


def swiglu(gu, out, n_rows=None):
    """out[t,j] = silu(gate)*up from the fused, 8-row interleaved product gu [T,2F]."""
    _cuda(gu, out)
    F = gu.shape[-1] // 2
    n = gu.numel() // (2 * F) if n_rows is None else n_rows
    _need(gu.is_contiguous() and out.is_contiguous() and out.dtype == gu.dtype and out.shape[-1] == F
          and out.numel() >= n * F and gu.numel() >= n * 2 * F, "swiglu: gu [T,2F], out [T,F], same dtype")
    _need(F % 8 == 0, f"swiglu: the feed-forward width {F} must be a multiple of 8")
    _check(_lib("elementwise").ab_swiglu(_p(gu), _p(out), _dt(gu), n, F, _stream()), "swiglu")
    return out


def attention_simt(qkv, out, k_pages, v_pages, block_table, tok_pos, tok_seq, n_tokens, H, K, D, scale,
                   window=0):
    """Attention of every token over its sequence's cached keys, 32-bit arithmetic.

    qkv [T,(H+2K)D] (the q part is read), out [T,H*D].
    """
    _cuda(qkv, out, k_pages, v_pages, block_table, tok_pos, tok_seq)
    _need(qkv.is_contiguous() and out.is_contiguous() and out.dtype == qkv.dtype and k_pages.dtype == qkv.dtype,
          "attention: q, out and cache must share one dtype and be contiguous")
    _need(out.numel() >= n_tokens * H * D, "attention: out too small")
    _need(0 < D <= 256, f"attention (32-bit kernel): head size {D} is outside 1..256")
    _i32(tok_pos, n_tokens, "tok_pos")
    _i32(tok_seq, n_tokens, "tok_seq")
    page_size = k_pages.shape[2]
    _need(tuple(k_pages.shape[1:]) == (K, page_size, D) and k_pages.shape == v_pages.shape
          and k_pages.is_contiguous() and v_pages.is_contiguous(), "attention: cache pages [n_pages,K,page,D]")
    _check(_lib("attention_simt").ab_attention_simt(
        _p(qkv), qkv.shape[-1], _p(out), _dt(qkv), _p(k_pages), _p(v_pages), _p(block_table),
        block_table.shape[1], _p(tok_pos), _p(tok_seq), n_tokens, H, K, D, page_size, ctypes.c_float(scale),
        int(window or 0), _stream()), "attention_simt")
    return out


def gemm_f32(a, w, out, bias=None, n_rows=None):
    """out[M,N] = a[M,K] @ w[N,K]^T (+ bias) in true float32 (CUDA-core FMA, fixed k order)."""
    _cuda(a, w, out, bias)
    _need(a.dtype == torch.float32 and w.dtype == torch.float32 and out.dtype == torch.float32,
          "gemm_f32 takes float32 tensors")
    K = a.shape[-1]
    M = a.numel() // K if n_rows is None else n_rows
    N = w.shape[0]
    _need(a.is_contiguous() and w.is_contiguous() and out.is_contiguous() and w.dim() == 2 and w.shape[1] == K
          and out.shape[-1] == N and out.numel() >= M * N and a.numel() >= M * K,
          "gemm_f32: a [M,K], w [N,K], out [M,N], contiguous")
    if bias is not None:
        _need(bias.dtype == torch.float32 and bias.numel() == N and bias.is_contiguous(), "gemm_f32: bias f32 [N]")
    _check(_lib("gemm_f32").ab_gemm_f32_nt(_p(a), K, _p(w), K, _p(bias), _p(out), N, M, N, K, _stream()),
           "gemm_f32")
    return out


GEMV_MAX_ROWS = 8           # up to here the skinny-matrix kernel is the fastest (measured per shape)
GEMV_NARROW_MAX_ROWS = 16   # ... and up to here for matrices of no more 16-row slabs than the GPU has SMs
DEFER_NORM = True           # steps of up to GEMV_MAX_ROWS rows: RMS norms run inside the products around them
#                             (2048x2048: 4.1 against 5.3 us for the library, 2048x8192: 12.2 against 13.2)
# 9 to 64 rows go to the library product: the tcgen05 product with the weights on the 128-row side
# (`gemm_tc(swap=True)`) was measured against it at every shape of the 1B and 8B sizes and lost (gate|up
# with the activation 15.7-20.4 against 14.2-15.5 us, the head 95-106 against 80-98 us): a tcgen05.mma
# costs the same whatever its N, so 16 to 64 columns waste it.
TC_PERSISTENT_MIN_ROWS = 1024   # from here the persistent tcgen05 product with the SwiGLU tail beats the library
#                                 product followed by the activation kernel (16384x2048: 57.9 against 57.8 us at
#                                 1,024 rows, 100 against 120 at 2,048, 190 against 235 at 4,096)
_SM_COUNT: dict = {}


def _sm_count(device) -> int:
    n = _SM_COUNT.get(device)
    if n is None:
        n = _SM_COUNT[device] = torch.cuda.get_device_properties(device).multi_processor_count
    return n


def gemv_bf16(x, w, out, bias=None, n_rows=None, swiglu=False, slices=None, start_early=True, owed=None,
              residual=None, norm_weight=None, activation="silu"):
    """out[:n] = x[:n] @ w^T (+ bias) for n <= 32 rows, bfloat16 x [M,K], w [N,K].

    out bfloat16 or float32 [M,N]; with `swiglu`, w is the 8-row interleaved gate|up
    matrix [2F,K] and out is bfloat16 [M,F] = act(gate) * up (`activation`: "silu", "relu",
    "gelu_tanh").  `start_early` off: the kernel is
    launched without programmatic dependent launch, i.e. after the kernel before it has ended (for
    the product that follows the decode attention, see csrc/launch.cuh).

    The RMS norm between two products without a kernel of its own (see csrc/gemv_bf16.cu):
    `owed` = (ss float32 [M, n_part], width, eps): x's rows still owe the division by
    sqrt(sum(ss[m]) / width + eps), which is applied to the sums.  `residual` (float32 [M,N]) with
    `norm_weight` (float32 [N]): the result is added to the residual in place, out becomes
    bf16(residual * norm_weight) and the partial sums of the residual's squares are returned as
    float32 [M, ceil(N / 16)] (the `ss` of the next product's `owed`).
    """
    _cuda(x, w, out, bias, residual, norm_weight)
    n = x.shape[0] if n_rows is None else n_rows
    K = x.shape[1]
    N = w.shape[0]
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.is_contiguous() and w.is_contiguous()
          and w.dim() == 2 and w.shape[1] == K and out.is_contiguous(), "gemv_bf16: x [M,K], w [N,K] bfloat16")
    if not (0 < n <= 32 and n <= x.shape[0] and n <= out.shape[0]):
        raise KernelError(f"gemv_bf16 takes 1..32 rows, got {n}")
    if K % 8:
        raise KernelError(f"gemv_bf16: the inner size {K} must be a multiple of 8")
    ss_out = None
    if swiglu:
        _need(residual is None, "gemv_bf16: the activation and the residual epilogue exclude each other")
        _need(N % 16 == 0 and out.dtype == torch.bfloat16 and out.shape[-1] == N // 2,
              "gemv_bf16 swiglu: w [2F,K] with F a multiple of 8, out bfloat16 [M,F]")
        epi = 2
    elif residual is not None:
        _need(out.shape[-1] == N and out.dtype == torch.bfloat16, "gemv_bf16 residual: out bfloat16 [M,N]")
        _need(residual.dtype == torch.float32 and residual.is_contiguous() and residual.shape[-1] == N
              and residual.numel() >= n * N, "gemv_bf16 residual: float32 [M,N]")
        _need(norm_weight is not None and norm_weight.dtype == torch.float32 and norm_weight.numel() == N
              and norm_weight.is_contiguous(), "gemv_bf16 residual: norm weight float32 [N]")
        ss_out = torch.empty((out.shape[0], -(-N // 16)), dtype=torch.float32, device=x.device)
        epi = 3
    else:
        _need(out.shape[-1] == N and out.dtype in (torch.bfloat16, torch.float32), "gemv_bf16: out [M,N]")
        epi = 1 if out.dtype == torch.float32 else 0
    if bias is not None:
        _need(bias.dtype == torch.float32 and bias.numel() == N and bias.is_contiguous(), "gemv_bf16: bias f32 [N]")
    ss_in, n_part, inv_width, eps = None, 0, 0.0, 0.0
    if owed is not None:
        ss_in, width, eps = owed
        _cuda(ss_in)
        _need(ss_in.dtype == torch.float32 and ss_in.dim() == 2 and ss_in.is_contiguous() and ss_in.shape[0] >= n
              and width > 0, "gemv_bf16: owed sums of squares float32 [M, n_part]")
        n_part, inv_width = ss_in.shape[1], 1.0 / width
    lib = _lib("gemv_bf16")
    if slices is None:
        slices = lib.ab_gemv_bf16_slices(N, K, _sm_count(x.device))
    partials = arrivals = None
    if slices > 1:
        slabs = -(-N // 16)
        partials = torch.empty(slabs * slices * 128 * (1 if n <= 8 else 2 if n <= 16 else 4), dtype=torch.float32,
                               device=x.device)
        arrivals = _arrival_counters(x.device, slabs)
    if not start_early:
        lib.ab_pdl_hold(1)
    try:
        _check(lib.ab_gemv_bf16_gated(_p(x), _p(w), _p(bias), _p(out), _p(partials), _p(arrivals), n, N, K,
                                      out.shape[-1], epi, slices, _p(ss_in), n_part, ctypes.c_float(inv_width),
                                      ctypes.c_float(eps), _p(residual), _p(norm_weight), _p(ss_out),
                                      GATE_ACTIVATIONS[activation], _stream()), "gemv_bf16")
    finally:
        if not start_early:
            lib.ab_pdl_hold(0)
    return out if ss_out is None else (out, ss_out)


def _prefill_tiles(ctx, G, device, rows=64):
    """Tiles of query tokens for the tensor-core prefill kernels: (sequence, first packed token),
    longest key ranges first; a tile has `rows` query rows = rows // G tokens.  Planned once per
    step, group size and tile height."""
    key = ("attention_tiles", G, rows)
    plan = ctx.extras.get(key)
    if plan is None:
        tpt = max(1, rows // G)
        tiles, start = [], 0
        for b, (q, kv) in enumerate(zip(ctx.host_q_lens, ctx.host_kv_lens)):
            for q0 in range(0, q, tpt):
                tiles.append((kv - q + min(q0 + tpt, q), b, start + q0))
            start += q
        tiles.sort(key=lambda x: -x[0])
        t = torch.tensor([[x[1] for x in tiles], [x[2] for x in tiles]], dtype=torch.int32).to(device)
        plan = (t[0].contiguous(), t[1].contiguous(), len(tiles), tpt)
        ctx.extras[key] = plan
    return plan


_ARRIVALS: dict = {}
_OUTGROWN: list = []      # scratch that was replaced by larger scratch: kept, since graphs captured earlier use it
DECODE_MAX_CLUSTER = 8           # chunks of one (sequence, head) that the decode attention merges in a cluster
USE_TCGEN05_ATTENTION = True     # prefill steps of 128 tokens or more, head size 64: the tcgen05 kernel


def _arrival_counters(device, n: int):
    """Zeroed int32 counters for the decode kernel's last-arrival merge.  Every launch leaves them
    zero again, so one buffer per device serves all launches (which run one after another in a
    stream).  It only grows outside a graph capture."""
    buf = _ARRIVALS.get(device)
    if buf is None or buf.numel() < n:
        if torch.cuda.is_current_stream_capturing():
            raise KernelError(f"attention: {n} arrival counters needed during graph capture, "
                              f"{0 if buf is None else buf.numel()} allocated before it")
        if buf is not None:
            _OUTGROWN.append(buf)        # captured graphs may still point at it
        buf = torch.zeros(max(n, 1 << 16), dtype=torch.int32, device=device)
        _ARRIVALS[device] = buf
    return buf


_DECODE_PLANS: dict = {}


def _decode_attention_plan(pairs: int, width: int, D: int, sms: int):
    """CTA size (`small` 0, 1, 2: the CTA halved that many times, 1, 2, 4 CTAs per SM) and the number of
    chunks per sequence for the decode attention of `pairs` (sequence, KV head, head tile) triples over
    block tables `width` pages wide: the pair with the least estimated time.  The estimate is
    waves x (launch + rounds x round) + cluster, in microseconds, with constants measured on a B200
    (batch 8 and 1 at contexts of 512 to 3,800 tokens, batch 32 to 256 at 512): a CTA's launch and merge
    1.5, a round of loads and products 2.2 / 2.2 / 2.4 for the three sizes, the cluster's launch and merge
    3.2 (a second round in the same CTA costs less than a cluster of two; rounds only run for keys
    that exist, which the estimate cannot know: ties go to fewer chunks and larger CTAs)."""
    key = (pairs, width, D, sms)
    plan = _DECODE_PLANS.get(key)
    if plan is None:
        lib = _lib("attention_mma")
        best = None
        for small in (0, 1, 2):
            cap = lib.ab_attention_decode_round_keys(D, small) / 64.0        # pages per round
            slots = sms << small
            for n in range(1, DECODE_MAX_CLUSTER + 1):
                if n > 1 and n > width:
                    break
                rounds = math.ceil(-(-width // n) / cap)
                waves = -(-pairs * n // slots)
                est = waves * (1.5 + rounds * (2.2, 2.2, 2.4)[small]) + (3.2 if n > 1 else 0.0)
                if best is None or est < best[0] - 1e-9:
                    best = (est, small, n)
        plan = _DECODE_PLANS[key] = (best[1], best[2])
    return plan


_STREAM_SCRATCH: dict = {}


def _stream_scratch(device, n_partial: int, n_counters: int):
    """Scratch of the streamed decode attention's merge through memory: partial outputs, their (maximum,
    sum) pairs and zeroed arrival counters (every launch leaves them zero).  One set per device, used by
    one launch after another in a stream; it only grows outside a graph capture."""
    have = _STREAM_SCRATCH.get(device)
    if have is None or have[0].numel() < n_partial or have[2].numel() < n_counters:
        if torch.cuda.is_current_stream_capturing():
            raise KernelError(f"attention: scratch for {n_partial} partial sums needed during graph capture, "
                              f"{0 if have is None else have[0].numel()} allocated before it")
        n_partial = max(n_partial, 1 << 22)
        if have is not None:
            _OUTGROWN.append(have)       # captured graphs may still point at it
        have = (torch.empty(n_partial, dtype=torch.float32, device=device),
                torch.empty(max(n_partial // 8, 1 << 16), dtype=torch.float32, device=device),
                torch.zeros(max(n_counters, 1 << 16), dtype=torch.int32, device=device))
        _STREAM_SCRATCH[device] = have
    return have


def attention_stream(qkv, out, cache, ctx, H, K, D, scale, window=0, rot=None, fuse=0, pages_per_cta=8,
                     merge="memory", ring=1):
    """Decode attention that streams the cache through a ring of pages filled by TMA
    (csrc/attention_stream.cu): head sizes 64 and 128, bfloat16.  A CTA takes `pages_per_cta` pages of
    one (sequence, KV head); the chunks of a sequence are merged in chunk order, through scratch memory
    (`merge` "memory") or inside a cluster of up to 8 ("cluster").  `ring`: 0 a short ring (four CTAs per
    processor), 1 the usual one (two), 2 a deep one (one).  `fuse` as for the other decode kernel: 1 rotates q, 2 also rotates k
    and appends k, v to the cache."""
    lib = _lib("attention_stream")
    k_pages, v_pages, table = cache.k, cache.v, cache.block_table
    _cuda(qkv, out, k_pages, v_pages, table)
    T = ctx.n_tokens
    _need(lib.ab_attention_stream_supports(H, K, D) == 1, f"attention_stream: head size {D} is not 64 or 128")
    _need(qkv.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and k_pages.dtype == torch.bfloat16
          and qkv.is_contiguous() and out.is_contiguous() and qkv.dim() == 2 and out.numel() >= T * H * D
          and qkv.shape[-1] >= (H + (2 * K if fuse == 2 else 0)) * D and qkv.shape[0] >= T,
          "attention_stream takes contiguous bfloat16 qkv [T,(H+2K)D], out [T,H*D]")
    _need(tuple(k_pages.shape[1:]) == (K, 64, D) and k_pages.shape == v_pages.shape and k_pages.is_contiguous()
          and v_pages.is_contiguous(), "attention_stream: cache pages [n_pages,K,64,D]")
    _need(table.dtype == torch.int32 and table.dim() == 2 and table.is_contiguous() and table.shape[0] >= T,
          "block_table must be contiguous int32 [B,W]")
    cos, sin, n_rot, pairing = rot if (rot is not None and fuse) else (None, None, 0, 0)
    if cos is not None:
        _cuda(cos, sin)
        _need(cos.dtype == torch.float32 and sin.dtype == torch.float32 and cos.is_contiguous()
              and sin.is_contiguous() and cos.shape == sin.shape and cos.shape[-1] == n_rot // 2 and n_rot % 16 == 0
              and n_rot <= D, "rope tables must be float32 [P, n_rot/2], n_rot a multiple of 16")
    _i32(ctx.tok_seq, T, "tok_seq")
    _i32(ctx.kv_len, T, "kv_len")
    order = getattr(ctx, "row_order", None)      # a permutation of the rows, longest sequence first
    if order is not None:
        _cuda(order)
        _i32(order, T, "row_order")
    width = max(int(table.shape[1]), 1)
    ppc = max(1, min(int(pages_per_cta), width))
    n_chunks = -(-width // ppc)
    kind = 0
    part_o = part_ml = arrivals = None
    if n_chunks > 1:
        if merge == "cluster" and n_chunks <= DECODE_MAX_CLUSTER:
            kind = 1
        else:
            kind = 2
            part_o, part_ml, arrivals = _stream_scratch(qkv.device, T * H * n_chunks * D, T * K * -(-(H // K) // 8))
    _tc_unchecked["attention_stream"] = True
    _check(lib.ab_attention_stream_bf16(
        _p(qkv), qkv.shape[-1], _p(out), _p(part_o), _p(part_ml), _p(arrivals), _p(k_pages), _p(v_pages),
        k_pages.shape[0], _p(table), table.shape[1], _p(ctx.tok_seq), _p(ctx.kv_len), _p(order), T, H, K, D,
        ctypes.c_float(scale), int(window or 0), ppc, n_chunks, kind, int(ring), _p(cos), _p(sin), n_rot,
        pairing, fuse, _stream()), "attention_stream")
    return out


STREAM_DECODE = True             # decode steps may take the streamed kernel (head sizes 64, 128)
STREAM_MIN_BYTES = None          # None: where it was measured to win (`_stream_pays`); a number: from that many
                                 # bytes of cache per layer, by the block table's width (0 always, inf never)


def _stream_pays(pairs: int, width: int, D: int) -> bool:
    """Whether the streamed decode attention beats the other decode kernel for `pairs` (sequence, KV head)
    pairs over block tables `width` pages wide.  Measured on a B200, each kernel with its own plan, 1 to 32
    sequences of 500 to 16,000 tokens, 8 and 32 KV heads (microseconds per layer, streamed / other): head
    size 128: it wins everywhere (one sequence of 500 tokens 6.1 / 7.8, 8 of 1,000 11.0 / 15.6, 2 of 16,000
    27 / 70); head size 64: it wins from tables of 24 pages (8 sequences of 2,000 tokens 11.0 / 14.0, 2 of 16,000
    16.8 / 33.2; a tie to 12 % worse for one or two sequences of 2,000 to 4,000), from 16 pages for up to
    four sequences (one of 1,000 tokens 5.4 / 7.3, four 6.7 / 8.1; eight are a tie at 1,000 tokens and
    lose at 800), and loses below (8 of 500 tokens 6.6 / 4.9, one 4.9 / 4.6) unless there are hundreds of
    pairs (32 sequences of 500: 9.0 / 10.1)."""
    if STREAM_MIN_BYTES is not None:
        return pairs * width * 64 * D * 4 >= STREAM_MIN_BYTES
    return D == 128 or width >= 24 or (width >= 16 and pairs <= 32) or pairs * width * 64 * D * 4 >= 30e6


def _stream_plan(rows: int, H: int, K: int, D: int, width: int, sms: int):
    """Whether the streamed decode attention should take a step of `rows` sequences whose block table is
    `width` pages wide, and how: None, or (pages per CTA, merge, ring).  Measured on a B200 against the
    other decode kernel at its best plan (microseconds per layer): 64 sequences of 530 tokens, 8 KV heads
    of 64: 15.4 against 17.5; of 2,000 tokens: 48.4 against 55.3; 64 sequences of 128 to 2,048 tokens, 8
    KV heads of 128: 63.1 against 100.9; 8 sequences of 16 to 1,024 tokens, 32 KV heads of 128: 17.9
    against 31.6; 8 sequences of 3,800 tokens, 8 heads of 64: 15.5 against 18.4.  Where little is read it loses
    at head size 64 (8 sequences of 640 tokens: 6.9 against 5.1; one sequence: 5.4 against 4.75), hence
    `_stream_pays`.  One CTA per (sequence, KV head) is best once there are more of those than processors;
    fewer are cut into chunks that a cluster merges; many CTAs of few pages take the short ring."""
    if not STREAM_DECODE or D not in (64, 128):
        return None
    pairs = rows * K * -(-(H // K) // 8)
    if not _stream_pays(pairs, width, D):
        return None
    want = -(-3 * sms // (2 * pairs))
    if want > DECODE_MAX_CLUSTER and width >= 8 * DECODE_MAX_CLUSTER:
        # few long sequences: more chunks than a cluster holds, merged through memory by the CTA that arrives
        # last, so that there are about 7/4 CTAs per processor, none with fewer than 4 pages (one sequence
        # of 30,000 tokens, 8 KV heads of 64: 18.9 us per layer with 32 chunks against 30.7 with a cluster's 8)
        chunks = max(1, min(-(-7 * sms // (4 * pairs)), width // 4, 64))
        return -(-width // chunks), "memory", 1
    chunks = max(1, min(DECODE_MAX_CLUSTER, want, width))
    ppc = -(-width // chunks)
    ring = 0 if (pairs * chunks > 2 * sms and ppc <= 16) else 1
    return ppc, "cluster", ring


def _attention_decode(qkv, out, cache, ctx, H, K, D, scale, window, rot=None, fuse=0):
    """Decode attention of one token per row of the batch: the kernel that fits the step's size."""
    plan = _stream_plan(ctx.n_tokens, H, K, D, max(int(cache.block_table.shape[1]), 1), _sm_count(qkv.device))
    if plan is not None:
        return attention_stream(qkv, out, cache, ctx, H, K, D, scale, window, rot, fuse, pages_per_cta=plan[0],
                                merge=plan[1], ring=plan[2])
    return _attention_decode_mma(qkv, out, cache, ctx, H, K, D, scale, window, rot, fuse)


def _attention_decode_mma(qkv, out, cache, ctx, H, K, D, scale, window, rot=None, fuse=0):
    """Decode attention: a CTA per (sequence, KV head, chunk of pages).  With few (sequence, head)
    pairs a CTA is large and a long table is cut into 2 to 8 chunks that are merged inside a
    thread-block cluster; with more pairs than processors the CTAs are smaller (several per
    processor) and each walks its whole table in rounds.
    `fuse` 1: the kernel also rotates q; 2: it rotates q and k and appends k, v to the cache."""
    lib = _lib("attention_mma")
    k_pages, v_pages, table = cache.k, cache.v, cache.block_table
    T = ctx.n_tokens
    cos, sin, n_rot, pairing = rot if (rot is not None and fuse) else (None, None, 0, 0)
    if cos is not None:
        _cuda(cos, sin)
        _need(cos.dtype == torch.float32 and sin.dtype == torch.float32 and cos.is_contiguous()
              and sin.is_contiguous() and cos.shape == sin.shape and cos.shape[-1] == n_rot // 2 and n_rot % 16 == 0
              and n_rot <= D, "rope tables must be float32 [P, n_rot/2], n_rot a multiple of 16")
    width = max(int(table.shape[1]), 1)
    small, n_chunks = _decode_attention_plan(T * K * -(-(H // K) // 8), width, D, _sm_count(qkv.device))
    pages_per_cta = -(-width // n_chunks)
    _i32(ctx.tok_seq, T, "tok_seq")
    _i32(ctx.kv_len, ctx.n_seqs, "kv_len")
    _check(lib.ab_attention_decode_rope_bf16(
        _p(qkv), qkv.shape[-1], _p(out), None, None, None, _p(k_pages), _p(v_pages), _p(table), table.shape[1],
        _p(ctx.tok_seq), _p(ctx.kv_len), T, H, K, D, ctypes.c_float(scale), int(window or 0), pages_per_cta,
        n_chunks, small, _p(cos), _p(sin), n_rot, pairing, fuse, _stream()), "attention_decode")
    return out


def attention_mma(qkv, out, cache, ctx, H, K, D, scale, window=0):
    """Tensor-core attention (bfloat16) over the paged cache; prefill or decode by the step's kind."""
    k_pages, v_pages, table = cache.k, cache.v, cache.block_table
    _cuda(qkv, out, k_pages, v_pages, table)
    T = ctx.n_tokens
    _need(qkv.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and k_pages.dtype == torch.bfloat16
          and qkv.is_contiguous() and out.is_contiguous(), "attention_mma takes contiguous bfloat16 tensors")
    _need(D % 16 == 0 and 0 < D <= 256 and H % K == 0 and H // K <= 64,
          f"attention_mma: head size {D} (multiples of 16 up to 256) or group size {H // K} (up to 64) not supported")
    _need(qkv.shape[-1] == (H + 2 * K) * D and out.numel() >= T * H * D, "attention_mma: qkv [T,(H+2K)D], out [T,H*D]")
    page = k_pages.shape[2]
    _need(page == 64 and tuple(k_pages.shape[1:]) == (K, 64, D) and k_pages.shape == v_pages.shape
          and k_pages.is_contiguous() and v_pages.is_contiguous(), "attention_mma: cache pages [n_pages,K,64,D]")
    lib = _lib("attention_mma")
    if ctx.is_decode:
        _i32(ctx.tok_seq, T, "tok_seq")
        return _attention_decode(qkv, out, cache, ctx, H, K, D, scale, window)
    _i32(ctx.tok_pos, T, "tok_pos")
    _i32(ctx.cu_q, ctx.n_seqs + 1, "cu_q")
    if USE_TCGEN05_ATTENTION and T >= 128 and qkv.shape[0] >= T:
        tc = _lib("attention_tc")
        if tc.ab_attention_prefill_tc_supports(H, K, D):
            _tc_unchecked["attention_tc"] = True
            tile_seq, tile_q0, n_tiles, _ = _prefill_tiles(ctx, H // K, qkv.device, rows=128)
            _check(tc.ab_attention_prefill_tc(
                _p(qkv), T, _p(out), _p(k_pages), _p(v_pages), k_pages.shape[0], _p(table), table.shape[1],
                _p(ctx.tok_pos), _p(ctx.cu_q), _p(tile_seq), _p(tile_q0), n_tiles, H, K, D, ctypes.c_float(scale),
                int(window or 0), _stream()), "attention_prefill_tc")
            return out
    tile_seq, tile_q0, n_tiles, tpt = _prefill_tiles(ctx, H // K, qkv.device)
    _check(lib.ab_attention_prefill_bf16(
        _p(qkv), qkv.shape[-1], _p(out), _p(k_pages), _p(v_pages), _p(table), table.shape[1], _p(ctx.tok_pos),
        _p(ctx.cu_q), _p(tile_seq), _p(tile_q0), n_tiles, tpt, H, K, D, ctypes.c_float(scale), int(window or 0),
        _stream()), "attention_prefill")
    return out


def attention(qkv, out, cache, ctx, H, K, D, scale, window=0):
    """Attention of the step's tokens over the paged cache (`cache`: a KVLayerView).

    bfloat16 with a head size in steps of 16 up to 256: the tensor-core kernels; everything
    else (the 32-bit path, other head sizes up to 256): the 32-bit kernel."""
    if qkv.dtype == torch.bfloat16 and D % 16 == 0 and D <= 256 and H // K <= 64:
        return attention_mma(qkv, out, cache, ctx, H, K, D, scale, window)
    return attention_simt(qkv, out, cache.k, cache.v, cache.block_table, ctx.tok_pos, ctx.tok_seq,
                          ctx.n_tokens, H, K, D, scale, window)


FUSE_ROPE_DECODE = True          # decode steps: rotation and append inside the attention kernel


def rope_attention(qkv, out, cache, ctx, H, K, D, scale, window=0, rot=None, write_cache=True):
    """Position rotation of q and k (`rot` = (cos, sin, n_rot, pairing) or None), append of k and v to
    the cache (unless `write_cache` is off: a layer that reads another layer's cache), then attention
    of the step's tokens over the cache.  Decode steps in bfloat16 do all of it in one kernel; everything else runs the rotation kernel and then `attention`."""
    cos, sin, n_rot, pairing = rot if rot is not None else (None, None, 0, 0)
    T = ctx.n_tokens
    max_len = getattr(ctx, "max_kv_len", None)
    if cos is not None and max_len is not None:
        _need(max_len <= cos.shape[0], f"rope tables hold {cos.shape[0]} positions, the step reaches position {max_len}")
    if (FUSE_ROPE_DECODE and ctx.is_decode and qkv.dtype == torch.bfloat16 and D % 16 == 0 and D <= 256
            and H // K <= 64 and n_rot % 16 == 0):
        _cuda(qkv, out, cache.k, cache.v, cache.block_table)
        _need(out.dtype == torch.bfloat16 and cache.k.dtype == torch.bfloat16 and qkv.is_contiguous()
              and out.is_contiguous() and qkv.shape[-1] == (H + 2 * K) * D and out.numel() >= T * H * D
              and H % K == 0, "rope_attention takes contiguous bfloat16 qkv [T,(H+2K)D], out [T,H*D]")
        _need(tuple(cache.k.shape[1:]) == (K, 64, D) and cache.k.shape == cache.v.shape and cache.k.is_contiguous()
              and cache.v.is_contiguous(), "rope_attention: cache pages [n_pages,K,64,D]")
        return _attention_decode(qkv, out, cache, ctx, H, K, D, scale, window, rot, 2 if write_cache else 1)
    rope_append(qkv, cos, sin, ctx.tok_pos, ctx.tok_seq, cache.block_table, cache.k, cache.v, T, H, K, D, n_rot,
                pairing, write_cache=write_cache, max_len=max_len)
    return attention(qkv, out, cache, ctx, H, K, D, scale, window)


def defers_norm(n_rows: int, width: int) -> bool:
    """Whether the product before a norm of a `width`-wide stream can leave `n_rows` rows prepared for
    the product after it (both must be the skinny product, see `gemv_bf16`)."""
    return DEFER_NORM and 0 < n_rows <= GEMV_MAX_ROWS and width % 8 == 0


def owed_norm_pays(n_rows: int, out_features: int, in_features: int, device) -> bool:
    """Whether the product [out_features, in_features] after a norm should finish the norm itself in a
    step of `n_rows` rows: only where its 16-row slabs are all resident at once (two CTAs per
    processor).  A grid of several waves loses more by the added tail of every CTA than the norm's
    kernel costs (measured, see csrc/gemv_bf16.cu)."""
    return (defers_norm(n_rows, in_features) and -(-out_features // 16) <= 2 * _sm_count(device))


def linear_bf16(x, w, out, n_rows=None, bias=None, start_early=True, owed=None):
    """out[:n] = x[:n] @ w^T (+ bias) for bfloat16 x [M,K], w [N,K]; out bfloat16 or float32 [M,N].

    Up to GEMV_MAX_ROWS rows (decode steps; GEMV_NARROW_MAX_ROWS for narrow matrices): the
    skinny-matrix kernel, which reads the weights once.  More rows: the library matrix product (as
    the reference uses BLAS)."""
    _cuda(x, w, out)
    n = x.shape[0] if n_rows is None else n_rows
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16, "linear_bf16 takes bfloat16 inputs")
    _need(x.dim() == 2 and w.dim() == 2 and x.shape[1] == w.shape[1] and out.shape[-1] == w.shape[0],
          "linear_bf16: x [M,K], w [N,K], out [M,N]")
    if x.shape[1] % 8 == 0 and (n <= GEMV_MAX_ROWS or (n <= GEMV_NARROW_MAX_ROWS
                                                       and -(-w.shape[0] // 16) <= _sm_count(x.device))):
        return gemv_bf16(x, w, out, bias=bias, n_rows=n, start_early=start_early, owed=owed)
    _need(owed is None, "linear_bf16: only the skinny product finishes a norm that its input owes")
    xs, ys = (x, out) if n == x.shape[0] == out.shape[0] else (x[:n], out[:n])
    if out.dtype == torch.float32:
        torch.mm(xs, w.t(), out_dtype=torch.float32, out=ys)
    else:
        torch.mm(xs, w.t(), out=ys)
    _mark("library product")
    if bias is not None:
        add_bias(ys, bias)
    return out


def repeat_penalty(logits, recent, penalty):
    """In place: for each distinct token of a row's window (int32 [B,R], -1 = unused),
    l > 0 -> l / penalty, else l * penalty."""
    _cuda(logits, recent)
    _need(logits.dtype == torch.float32 and logits.dim() == 2 and logits.is_contiguous(),
          "repeat_penalty: logits float32 [B,V]")
    _need(recent.dtype == torch.int32 and recent.dim() == 2 and recent.is_contiguous()
          and recent.shape[0] == logits.shape[0], "repeat_penalty: recent int32 [B,R]")
    _check(_lib("sampling").ab_repeat_penalty(_p(logits), _p(recent), logits.shape[0], recent.shape[1],
                                              logits.shape[1], ctypes.c_float(penalty), _stream()),
           "repeat_penalty")
    return logits


def sample(logits, out, temperature, top_k, top_p, seed, streams, steps, seed_dev=None):
    """One token per row of float32 logits [B,V] into out int32 [B].

    temperature <= 0: first index of the maximum.  Else top_k (<= 0: all), top_p
    (>= 1: all), and a draw with Philox(seed; stream, step) per row.  `seed_dev` (int32 [2]: low
    and high word, on the device) replaces `seed` when given.
    """
    _cuda(logits, out, streams, steps)
    _need(logits.dtype == torch.float32 and logits.dim() == 2 and logits.is_contiguous(),
          "sample: logits float32 [B,V]")
    B, V = logits.shape
    _i32(out, B, "out")
    _i32(streams, B, "streams")
    _i32(steps, B, "steps")
    if seed_dev is not None:
        _cuda(seed_dev)
        _i32(seed_dev, 2, "seed_dev")
    _check(_lib("sampling").ab_sample(_p(logits), B, V, _p(out), ctypes.c_float(temperature), int(top_k),
                                      ctypes.c_float(top_p), ctypes.c_uint64(int(seed) & (2**64 - 1)),
                                      _p(seed_dev), _p(streams), _p(steps), _stream()), "sample")
    return out


def decode_advance(tokens, tok_pos, kv_len, rng_step, tok_seq, sampled, recent, recent_pos, window,
                   history, counter, n_rows, host_ring=None):
    """Feeds the sampled tokens back as the next step's inputs (all int32, on the device); see the kernel.
    `host_ring`: pinned host memory int32 [R, rows]; the step's tokens are also written to its row
    counter % R, by the kernel itself."""
    _cuda(tokens, tok_pos, kv_len, rng_step, tok_seq, sampled, recent, recent_pos, history, counter)
    for t, name in ((tokens, "tokens"), (tok_pos, "tok_pos"), (kv_len, "kv_len"), (rng_step, "rng_step"),
                    (tok_seq, "tok_seq"), (sampled, "sampled")):
        _i32(t, n_rows, name)
    hist_len = 0
    if history is not None:
        _need(history.dtype == torch.int32 and history.is_contiguous() and history.shape[1] == n_rows
              and counter is not None and counter.dtype == torch.int32, "decode_advance: history int32 [L, rows]")
        hist_len = history.shape[0]
    if recent is not None:
        _need(recent.dtype == torch.int32 and recent.is_contiguous() and recent.numel() >= n_rows * window
              and recent_pos is not None, "decode_advance: recent int32 [rows, window]")
        _i32(recent_pos, n_rows, "recent_pos")
    ring_len = 0
    if host_ring is not None:
        _need(host_ring.device.type == "cpu" and host_ring.is_pinned() and host_ring.dtype == torch.int32
              and host_ring.is_contiguous() and host_ring.dim() == 2 and host_ring.shape[1] == n_rows
              and counter is not None, "decode_advance: host_ring pinned int32 [R, rows], with a counter")
        ring_len = host_ring.shape[0]
    _check(_lib("elementwise").ab_decode_advance(
        _p(tokens), _p(tok_pos), _p(kv_len), _p(rng_step), _p(tok_seq), _p(sampled), _p(recent), _p(recent_pos),
        int(window), _p(history), _p(counter), hist_len, _p(host_ring), ring_len, n_rows, _stream()),
        "decode_advance")


def gemm_tc(x, w, out, bias=None, n_rows=None, swiglu=False, swap=None, bn=None, slices=None, persistent=True,
            pair=None, activation="silu"):
    """out[:n] = x[:n] @ w^T (+ bias) on the tcgen05 tensor cores (TMA-fed, TMEM accumulators).

    x [M,K], w [N,K] bfloat16; out bfloat16 or float32 [M,N]; with `swiglu`, w is the 8-row
    interleaved gate|up matrix and out is bfloat16 [M, N/2] (`activation` on the gate: "silu"; "relu" and
    "gelu_tanh" in the persistent forms only).  `swap` puts the weights on the
    128-row side of the MMA (the batch, up to 256 rows, becomes the columns): the shape for decode
    steps.  `bn` is the MMA's column count per tile, `slices` the number of K slices.  Without `swap`,
    256-wide tiles and one slice run as the persistent kernel (one CTA per SM walks the tiles) unless
    `persistent` is off; `pair` chooses its form on pairs of processors (tiles of 256 x 256,
    `tcgen05.mma.cta_group::2`; default: `TC_PAIR`).
    """
    _cuda(x, w, out, bias)
    n = x.shape[0] if n_rows is None else n_rows
    K, N = x.shape[1], w.shape[0]
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.is_contiguous() and w.is_contiguous()
          and w.dim() == 2 and w.shape[1] == K and out.is_contiguous(), "gemm_tc: x [M,K], w [N,K] bfloat16")
    _need(K % 8 == 0, f"gemm_tc: the inner size {K} must be a multiple of 8")
    _need(x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0, "gemm_tc: operands must be 16-byte aligned")
    _need(0 < n <= x.shape[0] and n <= out.shape[0], "gemm_tc: row count")
    if swap is None:
        swap = n <= 64
    if bn is None:
        bn = (16 if n <= 16 else 32 if n <= 32 else 64 if n <= 64 else 128 if n <= 128 else 256) if swap else 256
    _need(bn in (16, 32, 64, 128, 256), "gemm_tc: bn must be 16, 32, 64, 128 or 256")
    if swiglu:
        _need(N % 16 == 0 and out.dtype == torch.bfloat16 and out.shape[-1] == N // 2,
              "gemm_tc swiglu: w [2F,K] with F a multiple of 8, out bfloat16 [M,F]")
        epi = 2 + GATE_ACTIVATIONS[activation]
        _need(epi == 2 or (not swap and bn == 256 and slices in (None, 1) and persistent),
              "gemm_tc: gates with another activation than SiLU run in the persistent forms only")
    else:
        _need(out.shape[-1] == N and out.dtype in (torch.bfloat16, torch.float32), "gemm_tc: out [M,N]")
        epi = 1 if out.dtype == torch.float32 else 0
    if bias is not None:
        _need(bias.dtype == torch.float32 and bias.numel() == N and bias.is_contiguous(), "gemm_tc: bias f32 [N]")
    _tc_unchecked["gemm_tc"] = True
    if not swap and bn == 256 and slices in (None, 1) and persistent:
        # many rows: the persistent form (tails under the next tile's main loop)
        lib = _lib("gemm_tc")
        run = lib.ab_gemm_tc_pair if (TC_PAIR if pair is None else pair) else lib.ab_gemm_tc_persistent
        _check(run(_p(x), _p(w), _p(bias), _p(out), n, N, K, out.shape[-1], epi, _stream()), "gemm_tc")
        return out
    rows_a, rows_b = (N, n) if swap else (n, N)
    tiles = -(-rows_a // 128) * -(-rows_b // bn)
    if slices is None:
        slices = max(1, min(-(-2 * _sm_count(x.device) // tiles), K // 1024)) if swap else 1
    partials = arrivals = None
    if slices > 1:
        partials = torch.empty(tiles * slices * 128 * bn, dtype=torch.float32, device=x.device)
        arrivals = _arrival_counters(x.device, tiles)
    _check(_lib("gemm_tc").ab_gemm_tc(_p(x), _p(w), _p(bias), _p(out), _p(partials), _p(arrivals), n, N, K,
                                      out.shape[-1], epi, 1 if swap else 0, bn, slices, _stream()), "gemm_tc")
    return out


# The persistent product on pairs of processors (`tcgen05.mma.cta_group::2`, see `gemm_tc`).  Measured on a
# B200 against the form with one processor per tile: gate|up with the activation 2048 x 16384 x 2048 101.6
# against 100.9 us, 4797 x 22016 x 4096 587 against 602, plain 16384 x 4096 x 14336 1,307 against 1,412 us
# (library 1,258); whole prompt steps: 1B shape 2,048 tokens 4.35 ms either way, the 7B workload's 4,797 tokens
# 55.0 against 56.2 ms, the 8B workload's 76,771 tokens 1.00 against 1.07 s (it moves a third less through the
# shared memory, which under the power cap is worth more than the kernel alone shows).
TC_PAIR = True

# kernels that wait on barriers with a limit, launched since the last check
_tc_unchecked = {"gemm_tc": False, "attention_tc": False, "attention_stream": False}


def check_tc_status() -> None:
    """Raises `KernelError` if a kernel that waits on barriers with a limit (the tcgen05 kernels, the
    streamed decode attention), launched since the last call, gave up a wait (its output is then
    unfinished).  Call it where the stream has just been synchronised: it reads one word per library
    from the device, and nothing when no such kernel ran."""
    for name, read in (("gemm_tc", gemm_tc_status), ("attention_tc", attention_tc_status),
                       ("attention_stream", attention_stream_status)):
        if _tc_unchecked[name]:
            _tc_unchecked[name] = False
            code = read()
            if code:
                raise KernelError(f"a kernel of {name} gave up waiting on a barrier (code {code}); "
                                  "the results of the steps since the last check are not valid")


def gemm_tc_status() -> int:
    """0, or the code left by a tcgen05 kernel that gave up waiting on a barrier (synchronises)."""
    return _lib("gemm_tc").ab_gemm_tc_status()


def attention_tc_status() -> int:
    """0, or the code left by a tcgen05 attention kernel that gave up waiting on a barrier (synchronises)."""
    return _lib("attention_tc").ab_attention_tc_status()


def attention_stream_status() -> int:
    """0, or the code left by a streamed decode attention kernel that gave up waiting on a barrier (synchronises)."""
    return _lib("attention_stream").ab_attention_stream_status()


# ---------------------------------------------------------------------------
# the matrix-memory recurrence, attention over a cached latent, routed experts

def mlstm_state_row(D: int, V: int) -> int:
    """Floats that one (sequence, head) of the matrix memory keeps: S [D, V], n [D], m, padded to 16 bytes."""
    return (D * V + D + 1 + 3) & ~3


def mlstm_step(proj, offsets, bias_i, bias_f, state, ctx, H, D, V, cap, qscale, norm_weight, eps, out,
               write_state=True):
    """The matrix-memory recurrence over the step's tokens, from each sequence's state to its new state.

    proj float32 [T, N]: one row per token with q | k | v | g | zi | zf at `offsets` (six column offsets);
    state float32 [slots, H, mlstm_state_row(D, V)]; out [T, H*V] of the activation dtype gets
    o / rms(o per head) * norm_weight * sigmoid(g).  Sequences, slots and padding rows are taken from the
    context's device arrays (cu_q, slots, tok_seq)."""
    _cuda(proj, bias_i, bias_f, state, norm_weight, out)
    T, B = ctx.n_tokens, ctx.n_seqs
    off_q, off_k, off_v, off_g, off_i, off_f = (int(o) for o in offsets)
    ld = proj.shape[-1]
    _need(proj.dtype == torch.float32 and proj.is_contiguous() and proj.numel() >= T * ld,
          "mlstm_step: proj must be contiguous float32 [T, N]")
    _need(max(off_q + H * D, off_k + H * D, off_v + H * V, off_g + H * V, off_i + H, off_f + H) <= ld,
          "mlstm_step: an offset reaches beyond the projected row")
    row = mlstm_state_row(D, V)
    _need(state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (H, row),
          f"mlstm_step: state must be contiguous float32 [slots, {H}, {row}]")
    for b in (bias_i, bias_f):
        _need(b.dtype == torch.float32 and b.numel() == H and b.is_contiguous(), "mlstm_step: gate biases float32 [H]")
    _need(norm_weight.dtype == torch.float32 and norm_weight.numel() == H * V and norm_weight.is_contiguous(),
          "mlstm_step: norm weight float32 [H*V]")
    _need(out.is_contiguous() and out.shape[-1] == H * V and out.numel() >= T * H * V, "mlstm_step: out [T, H*V]")
    _i32(ctx.cu_q, B + 1, "cu_q")
    _i32(ctx.slots, B, "slots")
    _i32(ctx.tok_seq, T, "tok_seq")
    coef = torch.empty((T, H, 3), dtype=torch.float32, device=proj.device)
    o_raw = torch.empty((T, H, V + 1), dtype=torch.float32, device=proj.device)
    _check(_lib("mlstm").ab_mlstm_step(
        _p(proj), ld, off_q, off_k, off_v, off_g, off_i, off_f, _p(bias_i), _p(bias_f), _p(state), row, H, D, V,
        _p(ctx.cu_q), _p(ctx.slots), _p(ctx.tok_seq), B, T, ctypes.c_float(cap), ctypes.c_float(qscale), _p(coef),
        _p(o_raw), _p(norm_weight), ctypes.c_float(eps), _p(out), _dt(out), 1 if write_state else 0, _stream()),
        "mlstm_step", kernels=3)
    return out


def latent_prep(x, Q, C, R, q_norm_weight, c_norm_weight, eps, rot, ctx, cache, cq_out, write_cache=True):
    """Per token of x float32 [T, Q + C + R]: cq_out = rmsnorm(x[:Q]) * q_norm_weight; the page row of the
    token's position gets [rmsnorm(x[Q:Q+C]) * c_norm_weight | x[Q+C:] rotated by position].
    `rot` = (cos, sin, n_rot, pairing) with pairing 0 (pairs (2i, 2i+1)), or None.  `cache.k`: pages
    [n_pages, 1, page, C + R] of the activation dtype."""
    pages, table = cache.k, cache.block_table
    cos, sin, n_rot, pairing = rot if rot is not None else (None, None, 0, 0)
    _cuda(x, q_norm_weight, c_norm_weight, cos, sin, pages, table, cq_out)
    T = ctx.n_tokens
    _need(x.dtype == torch.float32 and x.is_contiguous() and x.shape[-1] >= (Q + C + R if write_cache else Q)
          and x.numel() >= T * x.shape[-1], "latent_prep: x must be contiguous float32 [T, Q + C + R] ([T, Q] for a "
          "caller that writes no cache)")
    _need(pairing == 0, "latent_prep rotates pairs (2i, 2i+1) only")
    _need(n_rot <= R, f"latent_prep: {n_rot} rotated dims, the rotated part has {R}")
    for wt, n in ((q_norm_weight, Q), (c_norm_weight, C)):
        if wt is None and not write_cache and n == C:      # a caller that writes no cache norms no latent
            continue
        _need(wt.dtype == torch.float32 and wt.numel() == n and wt.is_contiguous(), "latent_prep: norm weights float32")
    if n_rot:
        _need(cos.dtype == torch.float32 and sin.dtype == torch.float32 and cos.is_contiguous() and sin.is_contiguous()
              and cos.shape == sin.shape and cos.shape[-1] == n_rot // 2, "rotation tables must be float32 [P, n_rot/2]")
        _need(ctx.max_kv_len <= cos.shape[0],
              f"rotation tables hold {cos.shape[0]} positions, the step reaches position {ctx.max_kv_len}")
    page = pages.shape[2]
    _need(pages.is_contiguous() and tuple(pages.shape[1:]) == (1, page, C + R) and pages.dtype == cq_out.dtype,
          "latent_prep: pages [n_pages, 1, page, C + R] of the activation dtype")
    _need(table.dtype == torch.int32 and table.dim() == 2 and table.is_contiguous()
          and ctx.max_kv_len <= table.shape[1] * page, "latent_prep: the block table does not cover the step")
    _need(cq_out.is_contiguous() and cq_out.shape[-1] == Q and cq_out.numel() >= T * Q, "latent_prep: cq_out [T, Q]")
    _i32(ctx.tok_pos, T, "tok_pos")
    _i32(ctx.tok_seq, T, "tok_seq")
    _check(_lib("latent_attention").ab_latent_prep(
        _p(x), x.shape[-1], Q, C, R, _p(q_norm_weight), _p(c_norm_weight), ctypes.c_float(eps), _p(cos), _p(sin), n_rot,
        _p(ctx.tok_pos), _p(ctx.tok_seq), _p(table), table.shape[1], page, _p(pages), _p(cq_out), _dt(cq_out), T,
        1 if write_cache else 0, _stream()), "latent_prep")
    return cq_out


def heads_matmul(a, a_head_stride, w, out, out_head_stride, n_tokens, tail=0, rot=None, ctx=None, tail_at=None):
    """out[t, h, :N] = w[h] @ a[t, h, :K] for w [H, N, K]; a [T, H * a_head_stride], out [T, H * out_head_stride].
    `tail` dims behind the K read ones are copied behind the N written ones, the first n_rot of them rotated by
    position in pairs (2i, 2i+1) (`rot` = (cos, sin, n_rot, 0), positions and padding rows from `ctx`)."""
    cos, sin, n_rot, pairing = rot if rot is not None else (None, None, 0, 0)
    _cuda(a, w, out, cos, sin)
    if w is None:                  # the tail alone, written `tail_at` dims into each head of `out`
        H, N, K = a.shape[-1] // a_head_stride, 0, a_head_stride - tail
        w = a
    else:
        H, N, K = w.shape
    tail_at = N if tail_at is None else int(tail_at)
    _need(w.is_contiguous() and a.is_contiguous() and out.is_contiguous(), "heads_matmul takes contiguous tensors")
    _need(a.shape[-1] == H * a_head_stride and K + tail <= a_head_stride and a.numel() >= n_tokens * a.shape[-1],
          "heads_matmul: a [T, H * a_head_stride]")
    _need(out.shape[-1] == H * out_head_stride and N <= tail_at and tail_at + tail <= out_head_stride
          and out.numel() >= n_tokens * out.shape[-1], "heads_matmul: out [T, H * out_head_stride]")
    _need(pairing == 0 and n_rot <= tail, "heads_matmul rotates pairs (2i, 2i+1) of the tail only")
    tok_pos = tok_seq = None
    if ctx is not None:
        tok_pos, tok_seq = ctx.tok_pos, ctx.tok_seq
        _i32(tok_pos, n_tokens, "tok_pos")
        _i32(tok_seq, n_tokens, "tok_seq")
    _need(n_rot == 0 or (tok_pos is not None and cos is not None and cos.dtype == torch.float32
                         and cos.shape[-1] == n_rot // 2 and ctx.max_kv_len <= cos.shape[0]),
          "heads_matmul: a rotated tail needs positions and tables that cover them")
    _check(_lib("latent_attention").ab_heads_matmul(
        _p(a), _dt(a), a.shape[-1], a_head_stride, _p(w), _dt(w), _p(out), _dt(out), out.shape[-1], out_head_stride,
        n_tokens, H, N, K, tail, tail_at, _p(cos), _p(sin), n_rot, _p(tok_pos), _p(tok_seq), _stream()), "heads_matmul")
    return out


def latent_attention_mma_supports(H, C, R, dtype) -> bool:
    """Whether `latent_attention_mma` takes these sizes: bfloat16, rows of C + R dims in steps of 16 up to 256,
    up to 64 heads (all heads of a token share its keys: they are the rows of one tile)."""
    return dtype == torch.bfloat16 and (C + R) % 16 == 0 and 0 < C + R <= 256 and 0 < H <= 64


def latent_attention_mma(q, out, cache, ctx, H, C, R, scale, sink=None, window=0):
    """The same attention on the tensor-core kernels of csrc/attention_mma.cu: the cached rows [c | r] are one
    key/value head of C + R dims that all H query heads share, the values are the rows themselves (the first C
    dims of a head's output are its weighted sum of c), and the sink joins the denominator in the kernels' last
    step.  q, out bfloat16 [T, H*(C+R)]."""
    pages, table = cache.k, cache.block_table
    _cuda(q, out, pages, table, sink)
    T, D = ctx.n_tokens, C + R
    _need(latent_attention_mma_supports(H, C, R, q.dtype), f"latent_attention_mma: {H} heads of {D} dims not supported")
    _need(out.dtype == torch.bfloat16 and pages.dtype == torch.bfloat16 and q.is_contiguous() and out.is_contiguous()
          and q.shape[-1] == H * D and out.shape[-1] == H * D and q.numel() >= T * H * D and out.numel() >= T * H * D,
          "latent_attention_mma: q, out bfloat16 [T, H*(C+R)]")
    _need(pages.is_contiguous() and tuple(pages.shape[1:]) == (1, 64, D), "latent_attention_mma: pages [n_pages, 1, 64, C+R]")
    _need(table.dtype == torch.int32 and table.dim() == 2 and table.is_contiguous()
          and ctx.max_kv_len <= table.shape[1] * 64, "latent_attention_mma: the block table does not cover the step")
    if sink is not None:
        _need(sink.dtype == torch.float32 and sink.numel() == H and sink.is_contiguous(), "sink must be float32 [H]")
    lib = _lib("attention_mma")
    if ctx.is_decode:
        width = max(int(table.shape[1]), 1)
        small, n_chunks = _decode_attention_plan(T * -(-H // 8), width, D, _sm_count(q.device))
        _i32(ctx.tok_seq, T, "tok_seq")
        _i32(ctx.kv_len, ctx.n_seqs, "kv_len")
        _check(lib.ab_attention_decode_sink_bf16(
            _p(q), H * D, _p(out), None, None, None, _p(pages), _p(pages), _p(table), table.shape[1], _p(ctx.tok_seq),
            _p(ctx.kv_len), T, H, 1, D, ctypes.c_float(scale), int(window or 0), -(-width // n_chunks), n_chunks, small,
            None, None, 0, 0, 0, _p(sink), _stream()), "latent_attention_decode")
        return out
    _i32(ctx.tok_pos, T, "tok_pos")
    _i32(ctx.cu_q, ctx.n_seqs + 1, "cu_q")
    tile_seq, tile_q0, n_tiles, tpt = _prefill_tiles(ctx, H, q.device)
    _check(lib.ab_attention_prefill_sink_bf16(
        _p(q), H * D, _p(out), _p(pages), _p(pages), _p(table), table.shape[1], _p(ctx.tok_pos), _p(ctx.cu_q),
        _p(tile_seq), _p(tile_q0), n_tiles, tpt, H, 1, D, ctypes.c_float(scale), int(window or 0), _p(sink), _stream()),
        "latent_attention_prefill")
    return out


LIBRARY_HEADS_MIN_ROWS = 17     # from here the per-head products of bfloat16 steps are library products


def heads_mm_library(a, a_head_stride, K, w, out, out_head_stride, n_tokens):
    """out[t, h, :N] = a[t, h, :K] @ w[h] for w [H, K, N], bfloat16, as one library product per head on strided
    views (steps of many rows, where the one-warp-per-output kernel would re-read the weights per token)."""
    H, _, N = w.shape
    av = a[:n_tokens].view(n_tokens, H, a_head_stride)
    ov = out[:n_tokens].view(n_tokens, H, out_head_stride)
    for h in range(H):
        torch.mm(av[:, h, :K], w[h], out=ov[:, h, :N])
    _mark("library product")
    return out


def latent_attention(q, out, cache, ctx, H, C, R, scale, sink=None, window=0):
    """Attention of every token over its sequence's cached latent rows [c | r] (see csrc/latent_attention.cu).
    q float32 [T, H*(C+R)] (keys' up-projection folded in), out float32 [T, H*C], sink float32 [H] or None."""
    pages, table = cache.k, cache.block_table
    _cuda(q, out, pages, table, sink)
    T = ctx.n_tokens
    _need(q.dtype == torch.float32 and out.dtype == torch.float32 and q.is_contiguous() and out.is_contiguous()
          and q.shape[-1] == H * (C + R) and out.shape[-1] == H * C and q.numel() >= T * H * (C + R)
          and out.numel() >= T * H * C, "latent_attention: q float32 [T, H*(C+R)], out float32 [T, H*C]")
    page = pages.shape[2]
    _need(pages.is_contiguous() and tuple(pages.shape[1:]) == (1, page, C + R),
          "latent_attention: pages [n_pages, 1, page, C + R]")
    _need(table.dtype == torch.int32 and table.dim() == 2 and table.is_contiguous()
          and ctx.max_kv_len <= table.shape[1] * page, "latent_attention: the block table does not cover the step")
    if sink is not None:
        _need(sink.dtype == torch.float32 and sink.numel() == H and sink.is_contiguous(), "sink must be float32 [H]")
    _need(C + R <= 1024, f"latent_attention: rows of {C + R} dims are outside 1..1024")
    _i32(ctx.tok_pos, T, "tok_pos")
    _i32(ctx.tok_seq, T, "tok_seq")
    _check(_lib("latent_attention").ab_latent_attention_simt_window(
        _p(q), _p(out), _p(pages), _dt(pages), _p(table), table.shape[1], _p(ctx.tok_pos), _p(ctx.tok_seq), _p(sink),
        T, H, C, R, page, ctypes.c_float(scale), int(window or 0), _stream()), "latent_attention")
    return out


MOE_ACTIVATIONS = {"gelu": 0, "silu": 1}


MOE_SCORES = {"softmax": None, "logit": 0, "sigmoid": 1}


def moe_route(h, router, n_tokens, groups, keep, top, scale, bias=None, score="softmax", correction=None, group_top=1,
              renorm=True):
    """(experts int32 [T, top], weights float32 [T, top]) of every token: softmax over all experts, the `keep`
    best of `groups` groups of neighbours, the `top` best experts of those, weights renormalised times `scale`.
    `bias` float32 [E] is added to the logits.  (One group, scale 1: the softmax over the chosen logits alone.)
    `score` "sigmoid" (or "logit"): the scores are sigmoid(z) (or z); the choice is made by score + `correction`
    (float32 [E], if given), a group's score is the sum of its `group_top` largest choice scores, and the weights are
    the chosen experts' scores without the correction, divided by their sum only if `renorm`."""
    _cuda(h, router, bias, correction)
    _need(score in MOE_SCORES, f"moe_route: score must be one of {tuple(MOE_SCORES)}")
    _need(score != "softmax" or (correction is None and group_top == 1 and renorm),
          "moe_route: the softmax router has no correction, takes a group's largest score and renormalises")
    if correction is not None:
        _need(correction.dtype == torch.float32 and correction.is_contiguous() and correction.numel() == router.shape[0],
              "moe_route: correction float32 [experts]")
    if bias is not None:
        _need(bias.dtype == torch.float32 and bias.is_contiguous() and bias.numel() == router.shape[0],
              "moe_route: bias float32 [experts]")
    E, width = router.shape
    _need(router.dtype == torch.float32 and router.is_contiguous(), "the router's matrix must be float32")
    _need(h.is_contiguous() and h.shape[-1] == width and h.numel() >= n_tokens * width, "moe_route: h [T, width]")
    _need(E <= 1024 and groups > 0 and E % groups == 0 and 0 < keep <= groups and 0 < top <= keep * (E // groups),
          f"moe_route: {E} experts in {groups} groups, {keep} kept, {top} chosen cannot be routed")
    idx = torch.empty((max(n_tokens, 1), top), dtype=torch.int32, device=h.device)
    wts = torch.empty((max(n_tokens, 1), top), dtype=torch.float32, device=h.device)
    z = torch.empty((max(n_tokens, 1), E), dtype=torch.float32, device=h.device)
    if score != "softmax":
        _need(group_top >= 1 and E // groups <= 128, "moe_route: groups of up to 128 experts, group_top >= 1")
        _check(_lib("moe").ab_moe_route_scores(
            _p(h), _dt(h), width, _p(router), _p(bias), _p(correction), n_tokens, width, E, groups, keep, int(group_top),
            top, MOE_SCORES[score], 1 if renorm else 0, ctypes.c_float(scale), _p(z), _p(idx), _p(wts), _stream()),
            "moe_route", kernels=2)
        return idx, wts
    _check(_lib("moe").ab_moe_route_bias(_p(h), _dt(h), width, _p(router), _p(bias), n_tokens, width, E, groups, keep,
                                         top, ctypes.c_float(scale), _p(z), _p(idx), _p(wts), _stream()),
           "moe_route", kernels=2)
    return idx, wts


MOE_ALL_EXPERTS_MIN_ROWS = 33      # from here a bfloat16 step runs every expert on every token in two library
#                                    products (weights of experts that were not chosen are zero) instead of reading
#                                    the chosen experts' rows once per (token, expert) pair


def moe_experts(h, w_up, w_down, idx, wts, out, n_tokens, activation="gelu", gate_up=None):
    """out[t] = sum_j wts[t, j] * W_down[idx[t, j]] @ act(W_up[idx[t, j]] @ h[t]); w_up [E, ff, width],
    w_down [width, E, ff] (the experts side by side), all of h's dtype.  Gated experts: `gate_up` [2, E, ff, width]
    holds the gates' matrices and then the up-projections (`w_up` is then gate_up[1]), and an expert is
    W_down (act(W_gate h) * (W_up h))."""
    _cuda(h, w_up, w_down, idx, wts, out, gate_up)
    E, ff, width = w_up.shape
    if gate_up is not None:
        _need(tuple(gate_up.shape) == (2, E, ff, width) and gate_up.is_contiguous() and gate_up.dtype == h.dtype
              and w_up.data_ptr() == gate_up[1].data_ptr(), "moe_experts: gate_up [2, E, ff, width] with w_up its second half")
    top = idx.shape[-1]
    _need(tuple(w_down.shape) == (width, E, ff) and w_up.is_contiguous() and w_down.is_contiguous()
          and w_up.dtype == h.dtype and w_down.dtype == h.dtype, "moe_experts: w_up [E, ff, width], w_down [width, E, ff]")
    _need(h.is_contiguous() and h.shape[-1] == width and out.is_contiguous() and out.shape[-1] == width
          and out.dtype == h.dtype and out.numel() >= n_tokens * width, "moe_experts: h, out [T, width] of one dtype")
    _i32(idx, n_tokens * top, "experts")
    _need(wts.dtype == torch.float32 and wts.is_contiguous() and wts.numel() >= n_tokens * top, "weights float32 [T, top]")
    if h.dtype == torch.bfloat16 and MOE_ALL_EXPERTS_MIN_ROWS <= n_tokens <= 65535:
        first = w_up if gate_up is None else gate_up
        cols = first.numel() // width                      # E * ff, or twice that: the gates, then the up-projections
        up = torch.empty((n_tokens, cols), dtype=h.dtype, device=h.device)
        torch.mm(h[:n_tokens], first.view(cols, width).t(), out=up)
        _mark("library product")
        _check(_lib("moe").ab_moe_weigh_all_gated(_p(up), _dt(up), _p(idx), _p(wts), n_tokens, top, ff, E,
                                                  MOE_ACTIVATIONS[activation], 0 if gate_up is None else 1, _stream()),
               "moe_weigh_all")
        torch.mm(up[:, :E * ff], w_down.view(width, E * ff).t(), out=out[:n_tokens])
        _mark("library product")
        return out
    act = torch.empty((max(n_tokens, 1) * top, ff), dtype=h.dtype, device=h.device)
    _check(_lib("moe").ab_moe_pairs_gated(_p(h), _dt(h), width, _p(w_up), _p(gate_up), _p(w_down), _p(idx), _p(wts),
                                          _p(act), _p(out), n_tokens, top, width, ff, E, MOE_ACTIVATIONS[activation],
                                          _stream()), "moe_experts", kernels=2)
    return out


# ---------------------------------------------------------------------------
# gated feed-forwards with other activations, linear attention with a fixed decay, attention with several score
# maps and values of their own size, small kernels on the residual stream

GATE_ACTIVATIONS = {"silu": 0, "relu": 1, "gelu_tanh": 2}


def gated_act(gu, out, activation="silu", n_rows=None):
    """out[t,j] = act(gate) * up from the fused, 8-row interleaved product gu [T,2F] (`swiglu` with a choice of
    activation: "silu", "relu", "gelu_tanh")."""
    _cuda(gu, out)
    _need(activation in GATE_ACTIVATIONS, f"gated_act: activation {activation!r} is not one of {tuple(GATE_ACTIVATIONS)}")
    F = gu.shape[-1] // 2
    n = gu.numel() // (2 * F) if n_rows is None else n_rows
    _need(gu.is_contiguous() and out.is_contiguous() and out.dtype == gu.dtype and out.shape[-1] == F
          and out.numel() >= n * F and gu.numel() >= n * 2 * F, "gated_act: gu [T,2F], out [T,F], same dtype")
    _need(F % 8 == 0, f"gated_act: the feed-forward width {F} must be a multiple of 8")
    _check(_lib("elementwise").ab_gated_act(_p(gu), _p(out), _dt(gu), n, F, GATE_ACTIVATIONS[activation], _stream()),
           "gated_act")
    return out


def linear_attention_max_dim() -> int:
    """The largest query/key size per head that `linear_attention_step` takes."""
    return 256


LINEAR_ATTENTION_STREAM_FROM = 32     # tokens per sequence (on average) from which a step takes the form for prompts
LINEAR_ATTENTION_PIECES = True        # few long sequences are cut into pieces that are walked side by side
LINEAR_ATTENTION_CTAS = 2048          # ... as many as give about this many CTAs, none shorter than 64 tokens


def _linear_attention_pieces(ctx, H, D, V, device):
    """The pieces of a prompt step for the linear attention's walk, or None where the sequences alone fill the
    device: (item_seq, item_t0, item_t1, n_items, seq_first, seq_count) as device arrays, planned once per step
    from the lengths (which belong to the shape of a captured step)."""
    if not LINEAR_ATTENTION_PIECES or ctx.host_q_lens is None:
        return None
    cols = _lib("linear_attention").ab_linear_attention_stream_cols(D)
    per_seq = H * -(-V // cols)
    want = -(-LINEAR_ATTENTION_CTAS // max(per_seq * ctx.n_seqs, 1))
    if want <= 1:
        return None
    piece = max(64, -(-(-(-max(ctx.host_q_lens) // want)) // 16) * 16)
    if max(ctx.host_q_lens) < 2 * piece:
        return None
    key = ("linear_attention_pieces", piece)
    plan = ctx.extras.get(key)
    if plan is None:
        seq, t0, t1, first, count, start = [], [], [], [], [], 0
        for b, q in enumerate(ctx.host_q_lens):
            first.append(len(seq))
            for at in range(0, q, piece):
                seq.append(b)
                t0.append(start + at)
                t1.append(start + min(at + piece, q))
            count.append(len(seq) - first[-1])
            start += q
        n = len(seq)
        flat = torch.tensor(seq + t0 + t1 + first + count, dtype=torch.int32).to(device)
        B = ctx.n_seqs
        plan = (flat[:n], flat[n:2 * n], flat[2 * n:3 * n], n, flat[3 * n:3 * n + B], flat[3 * n + B:3 * n + 2 * B])
        ctx.extras[key] = plan
    return plan


def linear_attention_step(proj, offsets, decay, state, ctx, H, D, V, norm_weight, eps, out, write_state=True,
                          activation=True, rot=None, k_scale=1.0, head_norm=False, gate="sigmoid"):
    """Linear attention with a fixed decay per head over the step's tokens, from each sequence's state to its
    new state (csrc/linear_attention.cu).

    proj float32 [T, N]: one row per token with zq | zk | zv | g at `offsets` (four column offsets, before the
    activation); decay float32 [H]; state float32 [slots, H, D, V]; out [T, H*V] of the activation dtype gets
    o / rms(o over all heads) * norm_weight * sigmoid(g).  `proj` is scratch: a long step leaves the activations
    in it.

    `activation` off: q, k, v enter as projected (on: silu).  `rot` = (cos, sin, n_rot, pairing): q and k are rotated
    by position.  `k_scale` multiplies k after the rotation.  `head_norm`: the root mean square is taken per head
    (`norm_weight` may then be None: no weight).  `gate`: "sigmoid" or "silu" of g."""
    cos, sin, n_rot, pairing = rot if rot is not None else (None, None, 0, 0)
    _cuda(proj, decay, state, norm_weight, out, cos, sin)
    _need(gate in ("sigmoid", "silu"), f"linear_attention_step: gate {gate!r} is not sigmoid or silu")
    _need(norm_weight is not None or head_norm, "linear_attention_step: the norm over all heads needs a weight")
    if cos is not None:
        _need(sin is not None and cos.dtype == torch.float32 and sin.dtype == torch.float32 and cos.is_contiguous()
              and sin.is_contiguous() and cos.shape == sin.shape and cos.shape[-1] == n_rot // 2 and n_rot % 2 == 0
              and 0 < n_rot <= D, "linear_attention_step: rope tables float32 [P, n_rot/2], n_rot even and at most D")
        _need(ctx.max_kv_len <= cos.shape[0],
              f"rope tables hold {cos.shape[0]} positions, the step reaches position {ctx.max_kv_len}")
        _i32(ctx.tok_pos, ctx.n_tokens, "tok_pos")
    T, B = ctx.n_tokens, ctx.n_seqs
    off_q, off_k, off_v, off_g = (int(o) for o in offsets)
    ld = proj.shape[-1]
    _need(proj.dtype == torch.float32 and proj.is_contiguous() and proj.numel() >= T * ld,
          "linear_attention_step: proj must be contiguous float32 [T, N]")
    _need(min(off_q, off_k, off_v, off_g) >= 0
          and max(off_q + H * D, off_k + H * D, off_v + H * V, off_g + H * V) <= ld,
          "linear_attention_step: an offset reaches beyond the projected row")
    _need(0 < D <= linear_attention_max_dim(), f"linear_attention_step: {D} dims per head are outside 1..256")
    _need(state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (H, D, V),
          f"linear_attention_step: state must be contiguous float32 [slots, {H}, {D}, {V}]")
    _need(decay.dtype == torch.float32 and decay.numel() == H and decay.is_contiguous(),
          "linear_attention_step: decay float32 [H]")
    _need(norm_weight is None or (norm_weight.dtype == torch.float32 and norm_weight.numel() == H * V
                                  and norm_weight.is_contiguous()), "linear_attention_step: norm weight float32 [H*V]")
    _need(out.is_contiguous() and out.shape[-1] == H * V and out.numel() >= T * H * V,
          "linear_attention_step: out [T, H*V]")
    _i32(ctx.cu_q, B + 1, "cu_q")
    _i32(ctx.slots, B, "slots")
    _i32(ctx.tok_seq, T, "tok_seq")
    o_raw = torch.empty((T, H * V), dtype=torch.float32, device=proj.device)
    long_step = T > LINEAR_ATTENTION_STREAM_FROM * B
    plan = _linear_attention_pieces(ctx, H, D, V, proj.device) if long_step else None
    item_seq, item_t0, item_t1, n_items, seq_first, seq_count = plan if plan is not None else (None,) * 3 + (0, None, None)
    pieces = torch.empty((n_items, H, D, V), dtype=torch.float32, device=proj.device) if n_items else None
    plain_qk = cos is None and k_scale == 1.0
    _check(_lib("linear_attention").ab_linear_attention_step_opts(
        _p(proj), ld, off_q, off_k, off_v, off_g, _p(decay), _p(state), H, D, V, _p(ctx.cu_q), _p(ctx.slots),
        _p(ctx.tok_seq), B, T, _p(o_raw), _p(norm_weight), ctypes.c_float(eps), _p(out), _dt(out),
        1 if write_state else 0, LINEAR_ATTENTION_STREAM_FROM, _p(item_seq), _p(item_t0), _p(item_t1), n_items,
        _p(pieces), _p(seq_first), _p(seq_count), 1 if activation else 0, _p(cos), _p(sin), int(n_rot), int(pairing),
        _p(ctx.tok_pos) if cos is not None else None, ctypes.c_float(k_scale), 1 if head_norm else 0,
        1 if gate == "silu" else 0, _stream()), "linear_attention_step",
        kernels=((4 if n_items else 2) + (1 if activation else 0) + (0 if plain_qk else 1)) if long_step else 2)
    return out


ATTENTION_MAPS_MAX_DIM = 256


def attention_prepare(buf, offsets, H, G, M, Dk, Dv, cache, ctx, q_weight=None, k_weight=None, eps=0.0, rot=None,
                      write_cache=True, bias=None, v_norm=False, v_side_by_side=False):
    """Query and key norm, position rotation and the append of keys and values to the cache, for an attention
    whose heads have M score maps (csrc/attention_maps.cu).

    buf [T, N]: per token H*M query vectors of Dk at offsets[0], G*M key vectors of Dk at offsets[1], G value
    vectors of Dv at offsets[2] (which may be the keys' own place: values that are the keys as projected).
    The queries are rewritten in place; keys and values go to `cache` (a KVLayerView whose key pages are
    [n_pages, G*M, page, Dk] and value pages [n_pages, G, page, Dv]).  `bias` float32 [N]: the projection's
    bias where the product left it out; it is added first.  `v_norm`: every value vector is divided by its root mean
    square (eps inside the root) before it is stored.  `v_side_by_side`: the value pages are [n_pages, 1, page,
    G*Dv], a token's value heads in one row."""
    k_pages, v_pages, table = cache.k, cache.v, cache.block_table
    cos, sin, n_rot, pairing = rot if rot is not None else (None, None, 0, 0)
    _cuda(buf, k_pages, v_pages, table, q_weight, k_weight, cos, sin)
    T = ctx.n_tokens
    off_q, off_k, off_v = (int(o) for o in offsets)
    N = buf.shape[-1]
    _need(buf.is_contiguous() and buf.numel() >= T * N and min(off_q, off_k, off_v) >= 0
          and max(off_q + H * M * Dk, off_k + G * M * Dk, off_v + G * Dv) <= N,
          "attention_prepare: buf [T, N] must hold the query, key and value vectors at their offsets")
    _need(0 < Dk <= ATTENTION_MAPS_MAX_DIM and 0 < Dv <= ATTENTION_MAPS_MAX_DIM,
          f"attention_prepare: head sizes {Dk}, {Dv} are outside 1..{ATTENTION_MAPS_MAX_DIM}")
    page = k_pages.shape[2]
    _need(k_pages.dtype == buf.dtype and v_pages is not None and v_pages.dtype == buf.dtype and k_pages.is_contiguous()
          and v_pages.is_contiguous() and tuple(k_pages.shape[1:]) == (G * M, page, Dk)
          and tuple(v_pages.shape[1:]) == ((1, page, G * Dv) if v_side_by_side else (G, page, Dv))
          and v_pages.shape[0] == k_pages.shape[0],
          f"attention_prepare: cache pages [n, {G * M}, page, {Dk}] and [n, {G}, page, {Dv}] of buf's dtype")
    _need(table.dtype == torch.int32 and table.dim() == 2 and table.is_contiguous()
          and ctx.max_kv_len <= table.shape[1] * page, "attention_prepare: the block table does not cover the step")
    for wgt in (q_weight, k_weight):
        if wgt is not None:
            _need(wgt.dtype == torch.float32 and wgt.numel() == Dk and wgt.is_contiguous(),
                  "attention_prepare: norm weights float32 [Dk]")
    if cos is not None:
        _need(sin is not None and cos.dtype == torch.float32 and sin.dtype == torch.float32 and cos.is_contiguous()
              and sin.is_contiguous() and cos.shape == sin.shape and cos.shape[-1] == n_rot // 2 and n_rot % 2 == 0
              and 0 < n_rot <= Dk, "attention_prepare: rope tables float32 [P, n_rot/2], n_rot even and at most Dk")
        _need(ctx.max_kv_len <= cos.shape[0],
              f"rope tables hold {cos.shape[0]} positions, the step reaches position {ctx.max_kv_len}")
    if bias is not None:
        _cuda(bias)
        _need(bias.dtype == torch.float32 and bias.numel() == N and bias.is_contiguous(),
              "attention_prepare: bias float32 [N]")
    _i32(ctx.tok_pos, T, "tok_pos")
    _i32(ctx.tok_seq, T, "tok_seq")
    _check(_lib("attention_maps").ab_attention_prepare_opts(
        _p(buf), _dt(buf), N, off_q, off_k, off_v, H * M, G * M, G, Dk, Dv, _p(q_weight), _p(k_weight),
        ctypes.c_float(eps), _p(cos), _p(sin), n_rot, pairing, _p(ctx.tok_pos), _p(ctx.tok_seq), _p(table),
        table.shape[1], _p(k_pages), _p(v_pages), page, T, 1 if write_cache else 0, _p(bias), 1 if v_norm else 0,
        1 if v_side_by_side else 0, _stream()), "attention_prepare")


def attention_maps(q, q_stride, out, cache, ctx, H, G, M, Dk, Dv, scale, window=0, sink=None, coef=0.0,
                   unit_norm=False, eps=0.0, out_scale=1.0):
    """Attention of every token over its sequence's cached keys and values, one warp per (token, head), 32-bit
    arithmetic (csrc/attention_maps.cu): M score maps per head, combined as a_0 + coef * (a_1 + ..), optionally
    divided by the head's root mean square, times `out_scale`.  q: the prepared rows (query vectors at the
    start of each row of `q_stride` elements); out [T, H*Dv] of q's dtype."""
    k_pages, v_pages, table = cache.k, cache.v, cache.block_table
    _cuda(q, out, k_pages, v_pages, table, sink)
    T = ctx.n_tokens
    _need(q.is_contiguous() and out.is_contiguous() and out.dtype == q.dtype and k_pages.dtype == q.dtype
          and v_pages.dtype == q.dtype and q.numel() >= T * q_stride and q_stride >= H * M * Dk
          and out.shape[-1] == H * Dv and out.numel() >= T * H * Dv,
          "attention_maps: q [T, stride], out [T, H*Dv] and the cache share one dtype")
    _need(0 < Dk <= ATTENTION_MAPS_MAX_DIM and 0 < Dv <= ATTENTION_MAPS_MAX_DIM and H % G == 0 and M >= 1,
          f"attention_maps: sizes {Dk}, {Dv} (1..{ATTENTION_MAPS_MAX_DIM}) or heads {H}/{G} not supported")
    page = k_pages.shape[2]
    _need(k_pages.is_contiguous() and v_pages.is_contiguous() and tuple(k_pages.shape[1:]) == (G * M, page, Dk)
          and tuple(v_pages.shape[1:]) == (G, page, Dv), "attention_maps: cache pages [n, G*M, page, Dk], [n, G, page, Dv]")
    _need(table.dtype == torch.int32 and table.dim() == 2 and table.is_contiguous()
          and ctx.max_kv_len <= table.shape[1] * page, "attention_maps: the block table does not cover the step")
    if sink is not None:
        _need(sink.dtype == torch.float32 and sink.numel() == H and sink.is_contiguous(), "sink must be float32 [H]")
    _i32(ctx.tok_pos, T, "tok_pos")
    _i32(ctx.tok_seq, T, "tok_seq")
    _check(_lib("attention_maps").ab_attention_maps(
        _p(q), q_stride, _p(out), _dt(q), _p(k_pages), _p(v_pages), _p(table), table.shape[1], _p(ctx.tok_pos),
        _p(ctx.tok_seq), T, H, G, M, Dk, Dv, page, ctypes.c_float(scale), int(window or 0), _p(sink),
        ctypes.c_float(coef), 1 if unit_norm else 0, ctypes.c_float(eps), ctypes.c_float(out_scale), _stream()),
        "attention_maps")
    return out


def attention_maps_mma_supports(H, G, M, Dk, Dv, stride, dtype) -> bool:
    """Whether `attention_maps_mma` takes these sizes (the tensor-core kernels of csrc/attention_mma.cu):
    bfloat16, key and value sizes in steps of 16 up to 256, up to 64 heads per key/value head, rows that start on
    16 bytes."""
    return (dtype == torch.bfloat16 and Dk % 16 == 0 and Dv % 16 == 0 and 0 < Dk <= 256 and 0 < Dv <= 256
            and H % G == 0 and H // G <= 64 and M >= 1 and stride % 8 == 0)


_ROW_INDEX: dict = {}


def _row_index(device, n: int):
    """int32 [0, 1, .., n-1] on the device (kept: captured steps read it again)."""
    key = (device.type, device.index)
    held = _ROW_INDEX.get(key)
    if held is None or held.numel() < n:
        if held is not None:
            _OUTGROWN.append(held)
        held = torch.arange(max(n, 1024), dtype=torch.int32, device=device)
        _ROW_INDEX[key] = held
    return held


def attention_maps_mma(q, q_stride, out, cache, ctx, H, G, M, Dk, Dv, scale, window=0, sink=None, coef=0.0,
                       unit_norm=False, eps=0.0, out_scale=1.0):
    """`attention_maps` on the tensor-core kernels (bfloat16 operands, float32 scores, softmax and sums): q holds
    the prepared query vectors at the start of each row, keys and values are in the cache already.  One map with
    equal key and value sizes in a step of one token each takes the decode kernel; everything else the kernel that
    tiles query rows (a step of one token each then has one token per tile).  Several maps leave their outputs
    in float32 and are combined by `ab_maps_combine`."""
    k_pages, v_pages, table = cache.k, cache.v, cache.block_table
    _cuda(q, out, k_pages, v_pages, table, sink)
    T = ctx.n_tokens
    _need(attention_maps_mma_supports(H, G, M, Dk, Dv, q_stride, q.dtype),
          f"attention_maps_mma: {H}/{G} heads, {M} maps of {Dk} and {Dv} dims not supported")
    _need(M > 1 or (not unit_norm and out_scale == 1.0), "attention_maps_mma: one map is left as it is attended")
    _need(out.dtype == torch.bfloat16 and k_pages.dtype == torch.bfloat16 and v_pages.dtype == torch.bfloat16
          and q.is_contiguous() and out.is_contiguous() and q.numel() >= T * q_stride and q_stride >= H * M * Dk
          and out.shape[-1] == H * Dv and out.numel() >= T * H * Dv, "attention_maps_mma: q [T, stride], out [T, H*Dv], bfloat16")
    _need(k_pages.is_contiguous() and v_pages.is_contiguous() and tuple(k_pages.shape[1:]) == (G * M, 64, Dk)
          and tuple(v_pages.shape[1:]) == (G, 64, Dv) and k_pages.shape[0] == v_pages.shape[0],
          "attention_maps_mma: cache pages [n_pages, G*M, 64, Dk] and [n_pages, G, 64, Dv]")
    _need(table.dtype == torch.int32 and table.dim() == 2 and table.is_contiguous()
          and ctx.max_kv_len <= table.shape[1] * 64, "attention_maps_mma: the block table does not cover the step")
    if sink is not None:
        _need(sink.dtype == torch.float32 and sink.numel() == H and sink.is_contiguous(), "sink must be float32 [H]")
    lib = _lib("attention_mma")
    _i32(ctx.tok_seq, T, "tok_seq")
    if ctx.is_decode and M == 1 and Dk == Dv:
        width = max(int(table.shape[1]), 1)
        small, n_chunks = _decode_attention_plan(T * G * -(-(H // G) // 8), width, Dk, _sm_count(q.device))
        _i32(ctx.kv_len, ctx.n_seqs, "kv_len")
        _check(lib.ab_attention_decode_sink_bf16(
            _p(q), q_stride, _p(out), None, None, None, _p(k_pages), _p(v_pages), _p(table), table.shape[1],
            _p(ctx.tok_seq), _p(ctx.kv_len), T, H, G, Dk, ctypes.c_float(scale), int(window or 0),
            -(-width // n_chunks), n_chunks, small, None, None, 0, 0, 0, _p(sink), _stream()), "attention_decode")
        return out
    _i32(ctx.tok_pos, T, "tok_pos")
    _i32(ctx.cu_q, ctx.n_seqs + 1, "cu_q")
    if (USE_TCGEN05_ATTENTION and not ctx.is_decode and M == 1 and Dk == Dv and Dk in (64, 128) and T >= 128
            and q.shape[0] >= T and q_stride % Dk == 0):
        tc = _lib("attention_tc")
        if tc.ab_attention_prefill_tc_supports(H, G, Dk):
            # long prompts, one map, head size 64 or 128: the tcgen05 kernel (a sink in its last step)
            _tc_unchecked["attention_tc"] = True
            tile_seq, tile_q0, n_tiles, _ = _prefill_tiles(ctx, H // G, q.device, rows=128)
            _check(tc.ab_attention_prefill_tc_sink(
                _p(q), q_stride // Dk, T, _p(out), _p(k_pages), _p(v_pages), k_pages.shape[0], _p(table), table.shape[1],
                _p(ctx.tok_pos), _p(ctx.cu_q), _p(tile_seq), _p(tile_q0), n_tiles, H, G, Dk, ctypes.c_float(scale),
                int(window or 0), _p(sink), _stream()), "attention_prefill_tc")
            return out
    if ctx.is_decode:
        # one token per sequence: a tile per token; the rows are the batch rows themselves
        tile_seq = tile_q0 = _row_index(q.device, T)
        n_tiles, tpt = T, 1
    else:
        tile_seq, tile_q0, n_tiles, tpt = _prefill_tiles(ctx, H // G, q.device)
    maps = out if M == 1 else torch.empty((q.shape[0], H * M * Dv), dtype=torch.float32, device=q.device)
    _check(lib.ab_attention_prefill_maps_bf16(
        _p(q), q_stride, _p(maps), 0 if M == 1 else 1, _p(k_pages), _p(v_pages), _p(table), table.shape[1],
        _p(ctx.tok_pos), _p(ctx.cu_q), _p(ctx.tok_seq), _p(tile_seq), _p(tile_q0), n_tiles, tpt, H * M, G * M, M, Dk, Dv,
        ctypes.c_float(scale), int(window or 0), _p(sink), _stream()), "attention_prefill")
    if M > 1:
        _check(_lib("attention_maps").ab_maps_combine(
            _p(maps), _p(out), _dt(out), _p(ctx.tok_seq), T, H, M, Dv, ctypes.c_float(coef),
            1 if unit_norm else 0, ctypes.c_float(eps), ctypes.c_float(out_scale), _stream()), "maps_combine")
    return out


def add_row(residual, row, ctx):
    """residual[t, :] += row[:] for every token of the step (float32)."""
    _cuda(residual, row)
    E, T = residual.shape[-1], ctx.n_tokens
    _need(residual.dtype == torch.float32 and residual.is_contiguous() and residual.numel() >= T * E
          and row.dtype == torch.float32 and row.is_contiguous() and row.numel() == E,
          "add_row: residual float32 [T, E], row float32 [E]")
    _i32(ctx.tok_seq, T, "tok_seq")
    _check(_lib("stream_ops").ab_add_row(_p(residual), _p(row), _p(ctx.tok_seq), T, E, _stream()), "add_row")
    return residual


def stream_cast(residual, delta, out, n_rows=None):
    """residual += delta (when given); out = residual in the activation dtype."""
    _cuda(residual, delta, out)
    E = residual.shape[-1]
    n = residual.numel() // E if n_rows is None else n_rows
    _need(residual.dtype == torch.float32 and residual.is_contiguous() and residual.numel() >= n * E
          and out.is_contiguous() and out.shape[-1] == E and out.numel() >= n * E,
          "stream_cast: residual float32 [T, E], out [T, E]")
    if delta is not None:
        _need(delta.is_contiguous() and delta.dtype == out.dtype and delta.shape[-1] == E and delta.numel() >= n * E,
              "stream_cast: delta [T, E] of out's dtype")
    _check(_lib("stream_ops").ab_stream_cast(_p(residual), _p(delta), _p(out), _dt(out), n, E, _stream()), "stream_cast")
    return out


def token_gate(z, table, offset, ctx, out):
    """out[t, j] = gelu_tanh(z[t, j]) * table[token_t, offset + j]; z, out [T, dim], table [V, W] of one dtype."""
    _cuda(z, table, out)
    T, dim = ctx.n_tokens, z.shape[-1]
    _need(z.is_contiguous() and out.is_contiguous() and table.is_contiguous() and table.dim() == 2
          and z.dtype == table.dtype == out.dtype and out.shape[-1] == dim and z.numel() >= T * dim
          and out.numel() >= T * dim and 0 <= offset and offset + dim <= table.shape[1],
          "token_gate: z, out [T, dim] and table [V, W] of one dtype, offset + dim <= W")
    _i32(ctx.tokens, T, "tokens")
    _i32(ctx.tok_seq, T, "tok_seq")
    _check(_lib("stream_ops").ab_token_gate(_p(z), _p(table), table.shape[1], int(offset), _p(ctx.tokens),
                                            _p(ctx.tok_seq), _p(out), _dt(z), T, dim, _stream()), "token_gate")
    return out


def add_unit_norm(residual, y, weight, eps, ctx):
    """residual[t, :] += y[t, :] / rms(y[t, :]) * weight for every token of the step (all float32)."""
    _cuda(residual, y, weight)
    E, T = residual.shape[-1], ctx.n_tokens
    _need(residual.dtype == torch.float32 and residual.is_contiguous() and residual.numel() >= T * E
          and y.dtype == torch.float32 and y.is_contiguous() and y.shape[-1] == E and y.numel() >= T * E
          and weight.dtype == torch.float32 and weight.is_contiguous() and weight.numel() == E,
          "add_unit_norm: residual, y float32 [T, E], weight float32 [E]")
    _i32(ctx.tok_seq, T, "tok_seq")
    _check(_lib("stream_ops").ab_add_unit_norm(_p(residual), _p(y), _p(weight), _p(ctx.tok_seq), T, E,
                                               ctypes.c_float(eps), _stream()), "add_unit_norm")
    return residual


# ---------------------------------------------------------------------------
# attention whose softmax weights are mixed across heads; sub-layers whose output is normed before it joins the stream

def talk_max_row() -> int:
    """The most numbers G*Dv of a token's values that `attention_talk` takes."""
    return 2048


TALK_ON_TENSOR_CORES = True      # bfloat16 steps whose sizes the tile kernel takes run there
TALK_DECODE_IN_PARTS = True      # steps of one token per sequence cut the keys into parts (`ab_talk_decode`)
TALK_DECODE_BLOCKS = 296         # CTAs that such a step aims at: two per processor
TALK_TILE_COLUMNS = 512          # columns of a token's value row that one launch of the tile kernel takes
TALK_GROUP_COLUMNS = 256         # of which a group of four warps takes this many (1, 2 or 4 groups per CTA)


def attention_talk(q, q_stride, out, cache, ctx, H, G, Dk, Dv, scale, talk, gate_rows=None, gate_stride=0, window=0):
    """Attention over the cached keys and values with the softmax weights mixed across heads:
    out[t, h] = gate * sum_g talk[h, g] * (weights of head g applied to the values of h's key/value head).

    q: the prepared rows, query vector x of a token at x*Dk, ordered so that vector x reads key head x % G (head
    g = (x % G) * (H/G) + x / G); cache: key pages [n, G, page, Dk], value pages [n, 1, page, G*Dv] (the heads of a
    token side by side); talk float32 [H, H]; gate_rows (or None): rows of `gate_stride` numbers of q's dtype whose
    first H*Dv are the gate's logits (sigmoid is applied); out [T, H*Dv] of q's dtype, heads in their own order.
    Every head's attention over all value heads is one float32 row A[t, x, G*Dv]; the mixing is a second kernel.
    In bfloat16 with sizes in steps of 16 the first is the tensor-core tile kernel, 256 columns of A per launch."""
    k_pages, v_pages, table = cache.k, cache.v, cache.block_table
    _cuda(q, out, k_pages, v_pages, table, talk, gate_rows)
    T, W = ctx.n_tokens, G * Dv
    page = k_pages.shape[2]
    _need(H % G == 0 and 0 < Dk <= ATTENTION_MAPS_MAX_DIM and 0 < W <= talk_max_row(),
          f"attention_talk: {H}/{G} heads of {Dk} and {Dv} dims not supported (G*Dv up to {talk_max_row()})")
    _need(q.is_contiguous() and out.is_contiguous() and out.dtype == q.dtype and k_pages.dtype == q.dtype
          and v_pages.dtype == q.dtype and q.numel() >= T * q_stride and q_stride >= H * Dk
          and out.shape[-1] == H * Dv and out.numel() >= T * H * Dv,
          "attention_talk: q [T, stride], out [T, H*Dv] and the cache share one dtype")
    _need(k_pages.is_contiguous() and v_pages.is_contiguous() and tuple(k_pages.shape[1:]) == (G, page, Dk)
          and tuple(v_pages.shape[1:]) == (1, page, W) and k_pages.shape[0] == v_pages.shape[0],
          "attention_talk: cache pages [n, G, page, Dk] and [n, 1, page, G*Dv]")
    _need(table.dtype == torch.int32 and table.dim() == 2 and table.is_contiguous()
          and ctx.max_kv_len <= table.shape[1] * page, "attention_talk: the block table does not cover the step")
    _need(talk.dtype == torch.float32 and talk.is_contiguous() and tuple(talk.shape) == (H, H),
          "attention_talk: talk float32 [H, H]")
    if gate_rows is not None:
        _need(gate_rows.dtype == q.dtype and gate_rows.is_contiguous() and gate_stride >= H * Dv
              and gate_rows.numel() >= (T - 1) * gate_stride + H * Dv, "attention_talk: gate rows of q's dtype")
    _i32(ctx.tok_pos, T, "tok_pos")
    _i32(ctx.tok_seq, T, "tok_seq")
    per = 8 if q.dtype == torch.bfloat16 else 4
    if TALK_DECODE_IN_PARTS and ctx.is_decode and page == 64 and Dk % per == 0 and W % 4 == 0:
        # one token per sequence: the keys in parts, so that few tokens fill the device.  The parts follow from the
        # block table's width alone (a captured step stays valid while its sequences grow)
        n_table = table.shape[1]
        if window:
            n_table = min(n_table, -(-int(window) // page) + 1)
        per_part = T * G * -(-(H // G) // 4) * -(-W // 512)
        parts = max(1, min(n_table, -(-TALK_DECODE_BLOCKS // per_part), 32))
        pages_per_part = -(-n_table // parts)
        parts = -(-n_table // pages_per_part)
        A = torch.empty((q.shape[0] * parts, H * W), dtype=torch.float32, device=q.device)
        ml = torch.empty((q.shape[0] * parts, H * 2), dtype=torch.float32, device=q.device)
        lib = _lib("attention_maps")
        _check(lib.ab_talk_decode(
            _p(q), q_stride, _p(A), _p(ml), parts, pages_per_part, _dt(q), _p(k_pages), _p(v_pages), _p(table),
            table.shape[1], _p(ctx.tok_pos), _p(ctx.tok_seq), T, H, G, Dk, Dv, page, ctypes.c_float(scale),
            int(window or 0), _stream()), "talk_decode")
        merged = torch.empty((q.shape[0], H * W), dtype=torch.float32, device=q.device)
        _check(lib.ab_talk_merge(_p(A), _p(ml), _p(merged), parts, T, H, W, _stream()), "talk_merge")
        _check(lib.ab_talk_combine(
            _p(merged), _p(talk), _p(gate_rows), int(gate_stride), _p(out), _dt(out), _p(ctx.tok_seq), T, H, G, Dv,
            _stream()), "talk_combine")
        return out
    A = torch.empty((q.shape[0], H * W), dtype=torch.float32, device=q.device)
    if (TALK_ON_TENSOR_CORES and page == 64 and W % 16 == 0
            and attention_maps_mma_supports(H // G, 1, G, Dk, min(W, TALK_GROUP_COLUMNS), q_stride, q.dtype)
            and H // G <= 64):
        # the tile kernel with the G key heads as the maps of one group whose value row is all heads' values; a launch
        # takes as many columns of that row as shared memory holds beside the keys (two tiles of each in flight), in
        # 1, 2 or 4 groups of warps
        _i32(ctx.cu_q, ctx.n_seqs + 1, "cu_q")
        if ctx.is_decode:
            tile_seq = tile_q0 = _row_index(q.device, T)
            n_tiles, tpt = T, 1
        else:
            tile_seq, tile_q0, n_tiles, tpt = _prefill_tiles(ctx, H // G, q.device)
        group = min(TALK_GROUP_COLUMNS, W)
        room = (227 * 1024 // 2 - 192 * (Dk + 8)) // 128 - 8          # value columns that fit beside the keys
        most = 4 if group <= 128 and Dk <= 128 else 2
        per_launch = max(group, min(TALK_TILE_COLUMNS, most * group, room // group * group))
        col0 = 0
        while col0 < W:
            cols = min(per_launch, W - col0)
            if -(-cols // group) == 3:      # 1, 2 or 4 groups: a third group's columns wait for the next launch
                cols = 2 * group
            _check(_lib("attention_mma").ab_attention_prefill_maps_groups_bf16(
                _p(q), q_stride, _p(A), 1, _p(k_pages), _p(v_pages), _p(table), table.shape[1], _p(ctx.tok_pos),
                _p(ctx.cu_q), _p(ctx.tok_seq), _p(tile_seq), _p(tile_q0), n_tiles, tpt, H, G, G, Dk, cols,
                ctypes.c_float(scale), int(window or 0), None, W, col0, group, _stream()), "attention_prefill")
            col0 += cols
    else:
        _check(_lib("attention_maps").ab_talk_attend(
            _p(q), q_stride, _p(A), _dt(q), _p(k_pages), _p(v_pages), _p(table), table.shape[1], _p(ctx.tok_pos),
            _p(ctx.tok_seq), T, H, G, Dk, Dv, page, ctypes.c_float(scale), int(window or 0), _stream()), "talk_attend")
    _check(_lib("attention_maps").ab_talk_combine(
        _p(A), _p(talk), _p(gate_rows), int(gate_stride), _p(out), _dt(out), _p(ctx.tok_seq), T, H, G, Dv, _stream()),
        "talk_combine")
    return out


def post_norm_add(residual, a, weight, eps, ctx=None, b=None, wa=None, wb=None, next_weight=None, out=None,
                  n_rows=None):
    """residual[t] += unit(y[t]) * weight with y = a, or y = (unit(a) * wa + unit(b) * wb) / 2 for two sub-layers side
    by side; then, if `out` is given, out[t] = unit(residual[t]) * next_weight in out's dtype.  unit(v) = v /
    sqrt(mean(v^2) + eps), 32-bit.  a, b [T, E] float32 or bfloat16; the weights float32 [E]."""
    _cuda(residual, a, b, weight, wa, wb, next_weight, out)
    E = residual.shape[-1]
    T = (ctx.n_tokens if ctx is not None else residual.numel() // E) if n_rows is None else n_rows
    _need(residual.dtype == torch.float32 and residual.is_contiguous() and residual.numel() >= T * E,
          "post_norm_add: residual float32 [T, E]")
    for t in (a, b):
        if t is not None:
            _need(t.is_contiguous() and t.shape[-1] == E and t.numel() >= T * E and t.dtype == a.dtype,
                  "post_norm_add: a and b [T, E] of one dtype")
    for w in (weight, wa, wb, next_weight):
        if w is not None:
            _need(w.dtype == torch.float32 and w.is_contiguous() and w.numel() == E, "post_norm_add: weights float32 [E]")
    _need((b is None) == (wa is None) == (wb is None), "post_norm_add: b comes with wa and wb")
    _need(E * 4 <= 200 * 1024, f"post_norm_add: rows of {E} numbers do not fit shared memory")
    if out is not None:
        _need(next_weight is not None and out.is_contiguous() and out.shape[-1] == E and out.numel() >= T * E,
              "post_norm_add: out [T, E] comes with next_weight")
    tok_seq = ctx.tok_seq if ctx is not None else None
    if tok_seq is not None:
        _i32(tok_seq, T, "tok_seq")
    _check(_lib("stream_ops").ab_post_norm_add(
        _p(residual), _p(a), _p(b), _dt(a), _p(wa), _p(wb), _p(weight), _p(next_weight), _p(out),
        _dt(out) if out is not None else 0, _p(tok_seq), T, E, ctypes.c_float(eps), _stream()), "post_norm_add")
    return out


# ---------------------------------------------------------------------------
# layer norm with weight and bias, an embedding with a factor and a table of token pairs, a gate per head, and
# recurrent mixers whose decay depends on the token (gated linear attention, the gated delta rule)

def layer_norm(residual, delta, weight, bias, eps, out, rows=None, n_rows=None):
    """Fused residual add and layer norm: residual += delta (when `rows` is None and delta is given);
    out[i] = (r - mean(r)) / sqrt(var(r) + eps) * weight + bias of row i (or row rows[i]) in out's dtype.
    residual float32 [T, E]; weight, bias float32 [E]; out None: the addition alone."""
    _cuda(residual, delta, weight, bias, out, rows)
    E = residual.shape[-1]
    T = residual.numel() // E
    _need(residual.dtype == torch.float32 and residual.is_contiguous(), "residual must be contiguous float32")
    for w in (weight, bias):
        _need(w.dtype == torch.float32 and w.numel() == E and w.is_contiguous(), "layer_norm: weight and bias float32 [E]")
    if delta is not None:
        _need(delta.is_contiguous() and delta.numel() == residual.numel(), "delta must match the residual")
    if rows is not None:
        n = rows.numel() if n_rows is None else n_rows
        _i32(rows, n, "rows")
    else:
        n = T if n_rows is None else n_rows
        _need(n <= T, "layer_norm: more rows than the residual has")
    _need(out is not None or delta is not None, "layer_norm needs delta or out")
    _need(E * 4 <= 200 * 1024, f"layer_norm: rows of {E} numbers do not fit shared memory")
    if out is not None:
        _need(out.is_contiguous() and out.numel() >= n * E, "layer_norm: out too small")
    _check(_lib("layer_norm").ab_layer_norm(
        _p(residual), _p(delta), _dt(delta) if delta is not None else 0, _p(rows), _p(weight), _p(bias), _p(out),
        _dt(out) if out is not None else 0, n, E, ctypes.c_float(eps), _stream()), "layer_norm")
    return out


def post_layer_norm_add(residual, a, weight, bias, eps, mult=1.0, ctx=None, b=None, ca=1.0, cb=1.0, next_weight=None,
                        next_bias=None, out=None, n_rows=None):
    """residual[t] += mult * LN(y[t]) with y = ca * a, or ca * a + cb * b for two sub-layers side by side, and LN the
    layer norm with `weight` and `bias`; then, if `out` is given, out[t] = LN_next(residual[t]) in out's dtype.
    a, b [T, E] float32 or bfloat16; weights and biases float32 [E]; 32-bit arithmetic."""
    _cuda(residual, a, b, weight, bias, next_weight, next_bias, out)
    E = residual.shape[-1]
    T = (ctx.n_tokens if ctx is not None else residual.numel() // E) if n_rows is None else n_rows
    _need(residual.dtype == torch.float32 and residual.is_contiguous() and residual.numel() >= T * E,
          "post_layer_norm_add: residual float32 [T, E]")
    for t in (a, b):
        if t is not None:
            _need(t.is_contiguous() and t.shape[-1] == E and t.numel() >= T * E and t.dtype == a.dtype,
                  "post_layer_norm_add: a and b [T, E] of one dtype")
    for w in (weight, bias, next_weight, next_bias):
        if w is not None:
            _need(w.dtype == torch.float32 and w.is_contiguous() and w.numel() == E,
                  "post_layer_norm_add: weights and biases float32 [E]")
    _need(E * 4 <= 200 * 1024, f"post_layer_norm_add: rows of {E} numbers do not fit shared memory")
    if out is not None:
        _need(next_weight is not None and next_bias is not None and out.is_contiguous() and out.shape[-1] == E
              and out.numel() >= T * E, "post_layer_norm_add: out [T, E] comes with the next norm's weight and bias")
    tok_seq = ctx.tok_seq if ctx is not None else None
    if tok_seq is not None:
        _i32(tok_seq, T, "tok_seq")
    _check(_lib("layer_norm").ab_post_layer_norm_add(
        _p(residual), _p(a), _p(b), _dt(a), ctypes.c_float(ca), ctypes.c_float(cb), _p(weight), _p(bias),
        ctypes.c_float(mult), _p(next_weight), _p(next_bias), _p(out), _dt(out) if out is not None else 0, _p(tok_seq),
        T, E, ctypes.c_float(eps), _stream()), "post_layer_norm_add")
    return out


def embed_pairs(table, scale, out, ctx, pairs=None, buckets=0, mul_prev=0, mul_cur=0, last_token=None):
    """out[t] = table[token_t] * scale (+ pairs[(prev_t * mul_prev + token_t * mul_cur) mod buckets], row `buckets` for
    a sequence's first token) as float32.  `last_token` int32 [slots, 1]: each sequence's last token so far, read for
    the step's first token of a sequence and set to its last."""
    _cuda(table, pairs, out, last_token)
    T, E = ctx.n_tokens, table.shape[1]
    _need(table.dim() == 2 and table.is_contiguous(), "embedding table must be contiguous [V, E]")
    _need(out.dtype == torch.float32 and out.is_contiguous() and out.shape[-1] == E and out.numel() >= T * E,
          "embed_pairs: out float32 [T, E]")
    _i32(ctx.tokens, T, "tokens")
    _i32(ctx.tok_seq, T, "tok_seq")
    if pairs is not None:
        _need(pairs.dtype == table.dtype and pairs.is_contiguous() and tuple(pairs.shape) == (buckets + 1, E),
              "embed_pairs: the pair table holds buckets + 1 rows of the embedding's width and dtype")
        _need(last_token is not None and last_token.dtype == torch.int32 and last_token.is_contiguous(),
              "embed_pairs: last_token int32 [slots]")
        _need(0 <= mul_prev < 2 ** 31 and 0 <= mul_cur < 2 ** 31 and buckets > 0, "embed_pairs: multipliers and buckets")
        _i32(ctx.tok_pos, T, "tok_pos")
        _i32(ctx.cu_q, ctx.n_seqs + 1, "cu_q")
        _i32(ctx.slots, ctx.n_seqs, "slots")
    _check(_lib("stream_ops").ab_embed_pairs(
        _p(table), _dt(table), ctypes.c_float(scale), _p(pairs), ctypes.c_longlong(buckets), ctypes.c_longlong(mul_prev),
        ctypes.c_longlong(mul_cur), _p(ctx.tokens), _p(ctx.tok_seq), _p(ctx.tok_pos), _p(ctx.cu_q), _p(ctx.slots),
        _p(last_token), _p(out), T, E, _stream()), "embed_pairs")
    return out


def head_gate(y, g, g_stride, n_tokens, H, V):
    """y[t, h, :] *= sigmoid(g[t * g_stride + h]) in place; y [T, H * V]; g: the gates' logits, one per head, in rows
    of `g_stride` numbers (a view into a wider product is fine)."""
    _cuda(y, g)
    _need(y.is_contiguous() and y.shape[-1] == H * V and y.numel() >= n_tokens * H * V, "head_gate: y [T, H * V]")
    _need(g_stride >= H and g.numel() >= (n_tokens - 1) * g_stride + H, "head_gate: g rows of g_stride >= H numbers")
    _check(_lib("stream_ops").ab_head_gate(_p(y), _dt(y), _p(g), _dt(g), int(g_stride), n_tokens, H, V, _stream()),
           "head_gate")
    return y


RECURRENCE_MAX_DIM = 256         # key dims per head that the walk holds in registers
RECURRENCE_ROUND = 8             # tokens of a sequence that the walk stages at a time (REC_TOKENS of the kernel)
RECURRENCE_CTAS = 296            # CTAs a walk aims at (two per processor): fewer value columns per CTA when few
#                                  (sequence, head) pairs would leave processors idle


def _recurrence_cols(n_seqs: int, H: int, V: int) -> int:
    for cols in (32, 16):
        if n_seqs * H * -(-V // cols) >= RECURRENCE_CTAS or V <= cols // 2:
            return cols
    return 8


def _f32_rows(t, n, name):
    _need(t.dtype == torch.float32 and t.stride(-1) == 1 and t.dim() == 2, f"{name}: float32 rows")
    return t.stride(0)


def gated_recurrence(mode, q, k, v, state, out, ctx, H, Hk, D, V, qscale=1.0, decay=None, beta=None, write_state=True):
    """One walk of a recurrent mixer over the step's tokens; q, k [T, Hk * D] and v [T, H * V] float32 (views with a
    row stride are fine), state float32 [slots, H, D, V], out float32 [T, H * V].
    mode "channel": S <- diag(a_t) S + k_t v_t^T, o_t = S^T (q_t qscale), decay a [T, H * D];
    mode "delta": S <- g_t S; u = beta_t (v_t - S^T k_t); S <- S + k_t u^T; o_t = S^T (q_t qscale), decay g and beta [T, H]."""
    _cuda(q, k, v, state, out, decay, beta)
    T = ctx.n_tokens
    _need(mode in ("channel", "delta"), "gated_recurrence: mode channel or delta")
    _need(0 < D <= RECURRENCE_MAX_DIM and H % Hk == 0, f"gated_recurrence: {D} dims per head are outside 1..{RECURRENCE_MAX_DIM}")
    ldq, ldk, ldv = _f32_rows(q, T, "q"), _f32_rows(k, T, "k"), _f32_rows(v, T, "v")
    _need(q.shape[0] >= T and k.shape[0] >= T and v.shape[0] >= T and q.shape[1] == Hk * D and k.shape[1] == Hk * D
          and v.shape[1] == H * V, "gated_recurrence: q, k [T, Hk * D], v [T, H * V]")
    _need(state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (H, D, V),
          "gated_recurrence: state float32 [slots, H, D, V]")
    _need(out.dtype == torch.float32 and out.is_contiguous() and out.shape[-1] == H * V and out.numel() >= T * H * V,
          "gated_recurrence: out float32 [T, H * V]")
    if mode == "channel":
        _need(decay is not None and decay.shape[0] >= T and decay.shape[1] == H * D, "gated_recurrence: decay [T, H * D]")
        ldd, dsc = _f32_rows(decay, T, "decay"), None
        dvec = decay
    else:
        for t in (decay, beta):
            _need(t is not None and t.dtype == torch.float32 and t.is_contiguous() and t.shape[-1] == H
                  and t.numel() >= T * H, "gated_recurrence: decay and beta float32 [T, H]")
        ldd, dvec, dsc = 0, None, decay
    _i32(ctx.cu_q, ctx.n_seqs + 1, "cu_q")
    _i32(ctx.slots, ctx.n_seqs, "slots")
    cols = _recurrence_cols(ctx.n_seqs, H, V)
    _check(_lib("gated_recurrence").ab_gated_recurrence(
        0 if mode == "channel" else 1, _p(q), ldq, _p(k), ldk, _p(v), ldv, _p(dvec), ldd, _p(dsc), _p(beta),
        ctypes.c_float(qscale), _p(state), _p(out), _p(ctx.cu_q), _p(ctx.slots), ctx.n_seqs, H, Hk, D, V, cols,
        1 if write_state else 0, 1 if ctx.max_q_len <= RECURRENCE_ROUND else 0, _stream()), "gated_recurrence")
    return out


def gla_decay(y, w2t, bias, tau, out, n_tokens):
    """out[t, c] = sigmoid(z)^(1/tau) with z = bias[c] + sum_r w2t[r, c] y[t, r]; y float32 rows of `rank` numbers (a
    view with a row stride is fine), w2t float32 [rank, channels] (the projection's matrix transposed), out float32
    [T, channels]."""
    w2 = w2t
    _cuda(y, w2, bias, out)
    rank, channels = w2.shape
    ldy = _f32_rows(y, n_tokens, "y")
    _need(y.shape[1] == rank and y.shape[0] >= n_tokens, "gla_decay: y [T, rank]")
    _need(w2.dtype == torch.float32 and w2.is_contiguous(), "gla_decay: w2t float32 [rank, channels]")
    if bias is not None:
        _need(bias.dtype == torch.float32 and bias.is_contiguous() and bias.numel() == channels, "gla_decay: bias float32")
    _need(out.dtype == torch.float32 and out.is_contiguous() and out.shape[-1] == channels and out.numel() >= n_tokens * channels,
          "gla_decay: out float32 [T, channels]")
    _need(tau > 0 and rank <= 1408, "gla_decay: tau positive, rank up to 1408")
    _check(_lib("gated_recurrence").ab_gla_decay(_p(y), ldy, _p(w2), _p(bias), ctypes.c_float(tau), _p(out), n_tokens,
                                                 channels, rank, _stream()), "gla_decay")
    return out


CONV_MAX_TAPS = 17


def gdr_prepare(x, taps_w, conv_state, A_log, dt_bias, b_off, a_off, qscale, unit_eps, qkv, beta, decay, ctx, H, G, D, V,
                write_state=True):
    """What the gated delta rule's walk reads, from the projected rows x float32 [T, ld] = [q | k | v | ...]: the short
    causal convolution per channel over time (taps_w float32 [2 G D + H V, taps], last column the token's own) with
    SiLU; q and k heads as unit vectors, q times qscale; beta = sigmoid(x[b_off + h]); decay = exp(-exp(A_log[h]) *
    softplus(x[a_off + h] + dt_bias[h])).  conv_state float32 [slots, taps - 1, channels]: a sequence's last inputs,
    read here and, if `write_state`, moved on by the step's."""
    _cuda(x, taps_w, conv_state, A_log, dt_bias, qkv, beta, decay)
    T = ctx.n_tokens
    Cc = 2 * G * D + H * V
    taps = taps_w.shape[1]
    _need(x.dtype == torch.float32 and x.is_contiguous() and x.dim() == 2 and x.shape[0] >= T
          and x.shape[1] >= max(Cc, b_off + H, a_off + H), "gdr_prepare: x float32 [T, ld]")
    _need(taps_w.dtype == torch.float32 and taps_w.is_contiguous() and taps_w.shape[0] == Cc and 1 <= taps <= CONV_MAX_TAPS,
          f"gdr_prepare: taps float32 [channels, 1..{CONV_MAX_TAPS}]")
    _need(conv_state.dtype == torch.float32 and conv_state.is_contiguous()
          and tuple(conv_state.shape[1:]) == (max(taps - 1, 1), Cc), "gdr_prepare: conv_state float32 [slots, taps - 1, channels]")
    for t in (A_log, dt_bias):
        _need(t.dtype == torch.float32 and t.is_contiguous() and t.numel() == H, "gdr_prepare: A_log, dt_bias float32 [H]")
    _need(qkv.dtype == torch.float32 and qkv.is_contiguous() and qkv.shape[-1] == Cc and qkv.numel() >= T * Cc,
          "gdr_prepare: qkv float32 [T, channels]")
    for t in (beta, decay):
        _need(t.dtype == torch.float32 and t.is_contiguous() and t.numel() >= T * H, "gdr_prepare: beta, decay float32 [T, H]")
    _need(Cc * 4 <= 200 * 1024, "gdr_prepare: a token's channels do not fit shared memory")
    _i32(ctx.tok_seq, T, "tok_seq")
    _i32(ctx.cu_q, ctx.n_seqs + 1, "cu_q")
    _i32(ctx.slots, ctx.n_seqs, "slots")
    _check(_lib("gated_recurrence").ab_gdr_prepare(
        _p(x), x.shape[1], _p(taps_w), taps, _p(conv_state), _p(A_log), _p(dt_bias), int(b_off), int(a_off),
        ctypes.c_float(qscale), ctypes.c_float(unit_eps), _p(qkv), _p(beta), _p(decay), _p(ctx.tok_seq), _p(ctx.cu_q),
        _p(ctx.slots), T, ctx.n_seqs, H, G, D, V, 1 if write_state else 0, _stream()), "gdr_prepare",
        kernels=2 if write_state and taps > 1 else 1)


HEAD_GATES = {None: 0, "silu": 1, "sigmoid": 2}


def head_norm_gate(o, weight, gate, gate_act, eps, out, ctx, H, V):
    """out[t, h, :] = o[t, h, :] / sqrt(mean(o[t, h, :]^2) + eps) * weight * act(gate[t, h, :]) in out's dtype; o float32
    [T, H * V], weight float32 [V] (one for all heads) or None, gate float32 rows of H * V numbers (a view with a row
    stride is fine) or None, act "silu" or "sigmoid"."""
    _cuda(o, weight, gate, out)
    T = ctx.n_tokens
    _need(o.dtype == torch.float32 and o.is_contiguous() and o.shape[-1] == H * V and o.numel() >= T * H * V,
          "head_norm_gate: o float32 [T, H * V]")
    if weight is not None:
        _need(weight.dtype == torch.float32 and weight.is_contiguous() and weight.numel() == V, "head_norm_gate: weight float32 [V]")
    ldg = 0
    if gate is not None:
        ldg = _f32_rows(gate, T, "gate")
        _need(gate.shape[0] >= T and gate.shape[1] == H * V and gate_act in ("silu", "sigmoid"), "head_norm_gate: gate [T, H * V]")
    _need(out.is_contiguous() and out.shape[-1] == H * V and out.numel() >= T * H * V, "head_norm_gate: out [T, H * V]")
    _i32(ctx.tok_seq, T, "tok_seq")
    _check(_lib("gated_recurrence").ab_head_norm_gate(
        _p(o), _p(weight), _p(gate), ldg, HEAD_GATES[gate_act if gate is not None else None], _p(out), _dt(out),
        _p(ctx.tok_seq), T, H, V, ctypes.c_float(eps), _stream()), "head_norm_gate")
    return out
