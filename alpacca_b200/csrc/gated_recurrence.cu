// Recurrent mixers whose state decays by amounts that depend on the token: one matrix S [D, V] per (sequence, head)
// in float32, carried from step to step.
//
//   mode 0, a decay per key channel (gated linear attention):
//       S <- diag(a_t) S + k_t v_t^T;   o_t = S^T (q_t * qscale)        a_t: D numbers in (0, 1) per head and token
//   mode 1, the gated delta rule:
//       S <- g_t S;   u = beta_t (v_t - S^T k_t);   S <- S + k_t u^T;   o_t = S^T q_t      g_t, beta_t: one number
//       per head and token; the read-out sees the token's own write
//
// The walk (`recurrence_kernel`): a CTA per (sequence, head, tile of value columns); a column's D entries are spread
// over 8, 16 or 32 neighbouring lanes' registers (a part of the rows each, read 16 bytes at a time), q, k and the decays of eight tokens at a time arrive in
// shared memory by `cp.async` through a ring of four buffers (three rounds' rows are on their way while one is walked), a
// column's dot products run in four chains per lane; the lanes' shares of a read-out wait in shared memory and are
// added after the round, so that the walk of a decay per channel has no exchange between lanes and no barrier in
// it (the delta rule needs one exchange per token, S^T k over all rows, by shuffles).  The order of additions depends
// on the column alone, so a token's output is bitwise the same in a prompt, a portion or a step of one token.
//
// Around it: `gla_decay` (a = sigmoid(z)^(1/tau) with z = W_2 y + b from the low-rank projection's first half y),
// `gdr_prepare` (a short causal convolution per channel over time with SiLU, whose last inputs are part of the
// state; q and k as unit vectors per head; beta = sigmoid; g = exp(-exp(A) softplus(a + dt))), and
// `head_norm_gate` (each head's output divided by its root mean square, times a weight per value channel, times
// SiLU or sigmoid of a gate).  All of it 32-bit arithmetic.
#include "common.cuh"
#include "launch.cuh"

#define REC_TOKENS 8        // tokens staged per round of the walk
#define REC_STAGES 4        // rounds whose rows are in flight or in use in a step of many tokens: the walk of a round is short
                            // against the memory's latency (a step of up to one round per sequence has one buffer)
#define CONV_MAX_TAPS 16

__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + expf(-x)); }

// 4 or 16 bytes from global to shared memory without passing registers; the copies of a round are one group
__device__ __forceinline__ void copy_async4(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src));
}
__device__ __forceinline__ void copy_async16(float* dst, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src));
}
__device__ __forceinline__ void copy_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void copy_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }


// Who copies what in a round: thread `tid` copies piece `c` (4 floats with 16-byte copies, else 1) of the rows of
// tokens tt = t_first, t_first + t_step, ..; worked out once, so that a round's copies cost no division.
struct RowCopier {
  int c, t_first, t_step;      // c < 0: this thread copies nothing
  __device__ __forceinline__ RowCopier(int pieces, int tid, int n_threads) {
    if (pieces <= 0) { c = -1; t_first = t_step = 1; return; }
    if (n_threads >= pieces) {
      t_step = n_threads / pieces;
      c = tid < t_step * pieces ? tid % pieces : -1;
      t_first = tid / pieces;
    } else {                     // more pieces than threads: every thread takes several of every row
      t_step = 1;
      t_first = 0;
      c = tid;
    }
  }
};

// rows of `n` tokens, `len` floats each, from `src + t * ld` to `dst + tt * pitch`.  With PART > 4 a row is laid out
// in parts of that many floats, each followed by four unused ones (element d at (d / PART) * (PART + 4) + d % PART),
// so that the lanes of a column, which each read their own part 16 bytes at a time, meet different banks.
template <int PART>
__device__ __forceinline__ void stage_rows(const RowCopier& w, float* dst, int pitch, const float* src, size_t ld, int n,
                                           int len, bool vec) {
  if (w.c < 0) return;
  const int pieces = vec ? len >> 2 : len;
  for (int c = w.c; c < pieces; c += blockDim.x) {
    const int d = vec ? c << 2 : c;
    const int at = PART > 4 ? (d / PART) * (PART + 4) + d % PART : d;
    for (int tt = w.t_first; tt < n; tt += w.t_step) {
      if (vec) copy_async16(dst + tt * pitch + at, src + (size_t)tt * ld + d);
      else copy_async4(dst + tt * pitch + at, src + (size_t)tt * ld + d);
    }
  }
}

// One token of one thread: its DR rows of column j.  Returns the thread's share of the read-out; the shares of a column's lanes are added after the round, so that a decay per channel needs no exchange
// between lanes while the tokens are walked.  The delta rule needs one per token: S^T k over all rows.
template <int DR, int LANES, int MODE>
__device__ __forceinline__ float walk_token(float (&S)[DR], const float4* __restrict__ qr, const float4* __restrict__ kr,
                                            const float4* __restrict__ ar, float vj, float g, float bt) {
  float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;      // four chains, added in a fixed order
  if (MODE == 0) {
#pragma unroll
    for (int i = 0; i < DR; i += 4) {
      const float4 a = ar[i >> 2], kk = kr[i >> 2], qq = qr[i >> 2];
      S[i] = a.x * S[i] + kk.x * vj;
      S[i + 1] = a.y * S[i + 1] + kk.y * vj;
      S[i + 2] = a.z * S[i + 2] + kk.z * vj;
      S[i + 3] = a.w * S[i + 3] + kk.w * vj;
      a0 += S[i] * qq.x;
      a1 += S[i + 1] * qq.y;
      a2 += S[i + 2] * qq.z;
      a3 += S[i + 3] * qq.w;
    }
  } else {
    float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;
#pragma unroll
    for (int i = 0; i < DR; i += 4) {
      const float4 kk = kr[i >> 2];
      S[i] *= g;
      S[i + 1] *= g;
      S[i + 2] *= g;
      S[i + 3] *= g;
      d0 += S[i] * kk.x;
      d1 += S[i + 1] * kk.y;
      d2 += S[i + 2] * kk.z;
      d3 += S[i + 3] * kk.w;
    }
    float dot = (d0 + d1) + (d2 + d3);
#pragma unroll
    for (int o = 1; o < LANES; o <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
    const float u = bt * (vj - dot);
#pragma unroll
    for (int i = 0; i < DR; i += 4) {
      const float4 kk = kr[i >> 2], qq = qr[i >> 2];
      S[i] += kk.x * u;
      S[i + 1] += kk.y * u;
      S[i + 2] += kk.z * u;
      S[i + 3] += kk.w * u;
      a0 += S[i] * qq.x;
      a1 += S[i + 1] * qq.y;
      a2 += S[i + 2] * qq.z;
      a3 += S[i + 3] * qq.w;
    }
  }
  return (a0 + a1) + (a2 + a3);
}

template <int DR, int LANES, int MODE, int STAGES>
__global__ void recurrence_kernel(const float* __restrict__ q, int ldq, const float* __restrict__ k, int ldk,
                                  const float* __restrict__ v, int ldv, const float* __restrict__ dvec, int ldd,
                                  const float* __restrict__ dsc, const float* __restrict__ beta, float qscale,
                                  float* __restrict__ state, float* __restrict__ out, const int* __restrict__ cu_q,
                                  const int* __restrict__ slots, int H, int Hk, int D, int V, int CV, int write_state,
                                  int vec) {
  extern __shared__ __align__(16) float rec_sm[];
  constexpr int DRP = DR > 4 ? DR + 4 : DR;     // a lane's part of a row, and the gap behind it
  constexpr int P4 = LANES * DRP;              // a token's row of q, k or decays
  pdl_wait();
  pdl_trigger();
  const int b = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * CV;
  const int slot = slots[b];
  if (slot < 0) return;
  const int kh = h / (H / Hk);
  const int tid = threadIdx.x, col = tid / LANES, r = tid % LANES;
  // a ring of buffers of a round's tokens: q, k (and the decays) of P4 floats each, CV values, two numbers per token
  constexpr int NV = MODE == 0 ? 3 : 2;
  const int per_buf = REC_TOKENS * (NV * P4 + CV + 4);
  float* shares = rec_sm + STAGES * per_buf;      // [REC_TOKENS][CV][LANES]: the lanes' shares of a round's read-outs
  float S[DR];                                 // rows r * DR .. r * DR + DR - 1 of column j
  float* st = state + ((size_t)slot * H + h) * D * V;
  // The tile of the state comes through shared memory: neighbouring threads fetch neighbouring columns of a row
  // (whole 32-byte pieces of memory), then every thread picks its rows.
  const int cv_shift = 31 - __clz(CV);         // CV is 8, 16 or 32
  for (int base = tid; base < D * CV; base += blockDim.x * 8) {      // eight loads in flight per thread
    float got[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int idx = base + u * blockDim.x;
      const int d = idx >> cv_shift, c = idx & (CV - 1);
      got[u] = (idx < D * CV && col0 + c < V) ? st[(size_t)d * V + col0 + c] : 0.f;
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int idx = base + u * blockDim.x;
      if (idx < D * CV) rec_sm[idx] = got[u];
    }
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < DR; ++i) {
    const int d = r * DR + i;
    S[i] = d < D ? rec_sm[d * CV + col] : 0.f;
  }
  __syncthreads();
  if (LANES * DR != D)                         // rows behind D are read as zeros
    for (int idx = tid; idx < STAGES * per_buf; idx += blockDim.x) rec_sm[idx] = 0.f;
  const int t0 = cu_q[b], t1 = cu_q[b + 1];
  const int cw = min(CV, V - col0);                        // this tile's columns
  const bool vec_v = vec && (cw & 3) == 0 && (col0 & 3) == 0;
  const RowCopier rows(vec ? D >> 2 : D, tid, blockDim.x), vals(vec_v ? cw >> 2 : cw, tid, blockDim.x);
  __syncthreads();
  auto stage = [&](int buf, int c0) {
    const int n = min(REC_TOKENS, t1 - c0);
    float* base = rec_sm + buf * per_buf;
    stage_rows<DR>(rows, base, P4, q + (size_t)c0 * ldq + (size_t)kh * D, ldq, n, D, vec);
    stage_rows<DR>(rows, base + REC_TOKENS * P4, P4, k + (size_t)c0 * ldk + (size_t)kh * D, ldk, n, D, vec);
    if (MODE == 0)
      stage_rows<DR>(rows, base + 2 * REC_TOKENS * P4, P4, dvec + (size_t)c0 * ldd + (size_t)h * D, ldd, n, D, vec);
    float* vs = base + NV * REC_TOKENS * P4;
    stage_rows<0>(vals, vs, CV, v + (size_t)c0 * ldv + (size_t)h * V + col0, ldv, n, cw, vec_v);
    if (MODE == 1 && tid < n) {
      float* sc = vs + REC_TOKENS * CV;
      copy_async4(sc + 2 * tid, dsc + (size_t)(c0 + tid) * H + h);
      copy_async4(sc + 2 * tid + 1, beta + (size_t)(c0 + tid) * H + h);
    }
    copy_commit();
  };
  // STAGES - 1 rounds are asked for before the first is walked; every turn of the loop commits one group (an
  // empty one once the tokens have run out), so that "all but the newest STAGES - 1" always covers the rows that the loop is about to walk
#pragma unroll
  for (int i = 0; i < STAGES - 1; ++i) {
    if (t0 + i * REC_TOKENS < t1) stage(i, t0 + i * REC_TOKENS);
    else copy_commit();
  }
  int buf = 0;
  for (int c0 = t0; c0 < t1; c0 += REC_TOKENS, buf = (buf + 1) % STAGES) {
    const int n = min(REC_TOKENS, t1 - c0);
    const int ahead = c0 + (STAGES - 1) * REC_TOKENS;
    if (ahead < t1) stage((buf + STAGES - 1) % STAGES, ahead);     // into the buffer that the round before left
    else copy_commit();
    copy_wait<STAGES - 1>();
    __syncthreads();
    const float* qs = rec_sm + buf * per_buf + r * DRP;
    const float* ks = qs + REC_TOKENS * P4;
    const float* as = ks + REC_TOKENS * P4;
    const float* vs = rec_sm + buf * per_buf + NV * REC_TOKENS * P4;
    const float* sc = vs + REC_TOKENS * CV;
    float* mine = shares + col * LANES + r;
    if (n == REC_TOKENS) {
      // a whole round: the shares wait in registers until its last token, so that no store stands between the loads
      // of one token and the next
      float sh[REC_TOKENS];
#pragma unroll
      for (int tt = 0; tt < REC_TOKENS; ++tt)
        sh[tt] = walk_token<DR, LANES, MODE>(S, reinterpret_cast<const float4*>(qs + tt * P4),
                                             reinterpret_cast<const float4*>(ks + tt * P4),
                                             reinterpret_cast<const float4*>(as + tt * P4), vs[tt * CV + col],
                                             MODE == 1 ? sc[2 * tt] : 0.f, MODE == 1 ? sc[2 * tt + 1] : 0.f);
#pragma unroll
      for (int tt = 0; tt < REC_TOKENS; ++tt) mine[tt * CV * LANES] = sh[tt];
    } else {
      for (int tt = 0; tt < n; ++tt)
        mine[tt * CV * LANES] = walk_token<DR, LANES, MODE>(S, reinterpret_cast<const float4*>(qs + tt * P4),
                                                            reinterpret_cast<const float4*>(ks + tt * P4),
                                                            reinterpret_cast<const float4*>(as + tt * P4), vs[tt * CV + col],
                                                            MODE == 1 ? sc[2 * tt] : 0.f, MODE == 1 ? sc[2 * tt + 1] : 0.f);
    }
    __syncthreads();
    // a column's read-out: its lanes' shares, added in lane order
    for (int idx = tid; idx < n * CV; idx += blockDim.x) {
      const int tt = idx / CV, c = idx - tt * CV;
      if (col0 + c >= V) continue;
      const float4* sh = reinterpret_cast<const float4*>(shares + (size_t)idx * LANES);
      float acc = 0.f;
#pragma unroll
      for (int i = 0; i < LANES / 4; ++i) {
        const float4 p = sh[i];
        acc += (p.x + p.y) + (p.z + p.w);
      }
      out[(size_t)(c0 + tt) * H * V + (size_t)h * V + col0 + c] = acc * qscale;
    }
  }
  if (!write_state) return;
  __syncthreads();                             // (every copy into the ring has landed: the last rounds asked for none)
#pragma unroll
  for (int i = 0; i < DR; ++i) {
    const int d = r * DR + i;
    if (d < D) rec_sm[d * CV + col] = S[i];
  }
  __syncthreads();
  for (int idx = tid; idx < D * CV; idx += blockDim.x) {
    const int d = idx >> cv_shift, c = idx & (CV - 1);
    if (col0 + c < V) st[(size_t)d * V + col0 + c] = rec_sm[idx];
  }
}

// One walk over the step's tokens.  q, k float32 rows with Hk heads of D (row strides ldq, ldk), v with H heads of V;
// mode 0: dvec [T, H * D] (row stride ldd); mode 1: dsc, beta [T, H].  state [slots, H, D, V]; out [T, H * V].
// `cols`: value columns per CTA (8, 16 or 32).  `one_round`: no sequence brings more than REC_TOKENS tokens.
AB_API int ab_gated_recurrence(int mode, const float* q, int ldq, const float* k, int ldk, const float* v, int ldv,
                               const float* dvec, int ldd, const float* dsc, const float* beta, float qscale, float* state,
                               float* out, const int* cu_q, const int* slots, int n_seqs, int H, int Hk, int D, int V,
                               int cols, int write_state, int one_round, cudaStream_t stream) {
  if (n_seqs <= 0) return AB_OK;
  if (H <= 0 || Hk <= 0 || H % Hk || D <= 0 || D > 256 || V <= 0 || (cols != 8 && cols != 16 && cols != 32)) return AB_BAD_ARG;
  if (!q || !k || !v || !state || !out || !cu_q || !slots) return AB_BAD_ARG;
  if (mode == 0 ? !dvec : (mode != 1 || !dsc || !beta)) return AB_BAD_ARG;
  // More lanes per column where few (sequence, head, column) triples would leave the schedulers with a warp or none
  // each: a walk is a chain of dependent steps per token, and what hides its latency is other warps.
  int lanes = 8;
  const long long threads8 = (long long)n_seqs * H * ((V + cols - 1) / cols) * cols * 8;
  if (mode == 0 && D > 32 && threads8 < 600LL * 32) lanes = 16;      // (the delta rule's lanes exchange a sum per token)
  const int per = (D + lanes - 1) / lanes;
  const int DR = per <= 4 ? 4 : (per <= 8 ? 8 : (per <= 16 ? 16 : 32));
  const int P4 = lanes * (DR > 4 ? DR + 4 : DR);
  const int stages = one_round ? 1 : REC_STAGES;
  const size_t smem = sizeof(float) * (stages * (size_t)REC_TOKENS * ((mode == 0 ? 3 : 2) * P4 + cols + 4) + (size_t)REC_TOKENS * cols * lanes);
  // 16-byte copies where every row starts on a 16-byte boundary
  auto al = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
  const int vec = (D % 4 == 0 && ldq % 4 == 0 && ldk % 4 == 0 && ldv % 4 == 0 && V % 4 == 0 && al(q) && al(k) && al(v) &&
                   (mode != 0 || (ldd % 4 == 0 && al(dvec)))) ? 1 : 0;
  const dim3 grid((unsigned)n_seqs, (unsigned)H, (unsigned)((V + cols - 1) / cols));
  const dim3 block((unsigned)(cols * lanes));
  bool done = false;
#define AB_GO(DRV, L, M, ST)                                                                                              \
  if (!done && DR == DRV && lanes == L && mode == M && stages == ST) {                                                    \
    if (smem > 48 * 1024)                                                                                                 \
      cudaFuncSetAttribute(recurrence_kernel<DRV, L, M, ST>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);     \
    ab_launch(recurrence_kernel<DRV, L, M, ST>, grid, block, smem, stream, q, ldq, k, ldk, v, ldv, dvec, ldd, dsc, beta,  \
              qscale, state, out, cu_q, slots, H, Hk, D, V, cols, write_state, vec);                                      \
    done = true;                                                                                                          \
  }
#define AB_BOTH(DRV, L) AB_GO(DRV, L, 0, 1) AB_GO(DRV, L, 1, 1) AB_GO(DRV, L, 0, REC_STAGES) AB_GO(DRV, L, 1, REC_STAGES)
  AB_BOTH(4, 8) AB_BOTH(8, 8) AB_BOTH(16, 8) AB_BOTH(32, 8)
  AB_BOTH(4, 16) AB_BOTH(8, 16) AB_BOTH(16, 16)
  AB_BOTH(4, 32) AB_BOTH(8, 32)
#undef AB_BOTH
#undef AB_GO
  if (!done) return AB_BAD_ARG;
  return ab_launch_status();
}

// a[t, c] = sigmoid(z)^(1/tau), z = b[c] + sum_r W2[c, r] y[t, r]; y: `rank` numbers per token at y + t * ldy; W2 is
// given transposed, [rank, channels], so that neighbouring threads read neighbouring numbers.
// A block of 32 channels x 8 tokens; its four warps each take a quarter of the rank (so that a step of a few tokens
// still spreads over many blocks and no thread walks the whole rank), and the quarters are added in order.
__global__ void __launch_bounds__(128)
gla_decay_kernel(const float* __restrict__ y, int ldy, const float* __restrict__ w2t, const float* __restrict__ bias,
                 float inv_tau, float* __restrict__ a, int n_tokens, int channels, int rank) {
  extern __shared__ float ys[];              // [8][rank]
  __shared__ float part[4][8][32];
  pdl_wait();
  pdl_trigger();
  const int t0 = blockIdx.y * 8, n = min(8, n_tokens - t0);
  for (int idx = threadIdx.x; idx < n * rank; idx += blockDim.x) {
    const int tt = idx / rank, rr = idx - tt * rank;
    ys[idx] = y[(size_t)(t0 + tt) * ldy + rr];
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, quarter = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + lane;
  const int span = (rank + 3) >> 2, r0 = quarter * span, r1 = min(rank, r0 + span);
  float z[8];
#pragma unroll
  for (int tt = 0; tt < 8; ++tt) z[tt] = 0.f;
  if (c < channels)
    for (int rr = r0; rr < r1; ++rr) {
      const float w = w2t[(size_t)rr * channels + c];
#pragma unroll
      for (int tt = 0; tt < 8; ++tt)
        if (tt < n) z[tt] += w * ys[tt * rank + rr];
    }
#pragma unroll
  for (int tt = 0; tt < 8; ++tt) part[quarter][tt][lane] = z[tt];
  __syncthreads();
  if (c >= channels) return;
  const float bc = bias != nullptr ? bias[c] : 0.f;
#pragma unroll
  for (int k = 0; k < 2; ++k) {                // warp w finishes tokens 2w and 2w + 1
    const int tt = quarter * 2 + k;
    if (tt < n) {
      const float zz = bc + ((part[0][tt][lane] + part[1][tt][lane]) + (part[2][tt][lane] + part[3][tt][lane]));
      a[(size_t)(t0 + tt) * channels + c] = expf(-softplus_f(-zz) * inv_tau);      // log sigmoid(z) = -softplus(-z)
    }
  }
}

AB_API int ab_gla_decay(const float* y, int ldy, const float* w2t, const float* bias, float tau, float* a, int n_tokens,
                        int channels, int rank, cudaStream_t stream) {
  if (n_tokens <= 0) return AB_OK;
  if (!y || !w2t || !a || channels <= 0 || rank <= 0 || !(tau > 0.f) || (size_t)rank * 32 > 44 * 1024) return AB_BAD_ARG;
  const dim3 grid((unsigned)((channels + 31) / 32), (unsigned)((n_tokens + 7) / 8));
  ab_launch(gla_decay_kernel, grid, dim3(128), (size_t)8 * rank * sizeof(float), stream, y, ldy, w2t, bias, 1.0f / tau, a,
            n_tokens, channels, rank);
  return ab_launch_status();
}

// Per token: the convolution over the token's and the `taps - 1` inputs before it, per channel, of the first `Cc` =
// 2 * G * D + H * V numbers of a projected row (q | k | v), then SiLU; q and k heads as unit vectors (x / sqrt(sum x^2
// + unit_eps)), q times qscale; beta = sigmoid(row[b_off + h]); g = exp(-exp(A[h]) * softplus(row[a_off + h] + dt[h])).
// Inputs from before the step come from `conv_state` [slots, taps - 1, Cc] (oldest first; zero at a sequence's start).
__global__ void gdr_prepare_kernel(const float* __restrict__ x, int ld, const float* __restrict__ taps_w, int taps,
                                   const float* __restrict__ conv_state, const float* __restrict__ A_log,
                                   const float* __restrict__ dt_bias, int b_off, int a_off, float qscale, float unit_eps,
                                   float* __restrict__ qkv, float* __restrict__ beta, float* __restrict__ decay,
                                   const int* __restrict__ tok_seq, const int* __restrict__ cu_q,
                                   const int* __restrict__ slots, int H, int G, int D, int V) {
  extern __shared__ float cv[];              // [Cc]
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  const int b = tok_seq[t];
  if (b < 0) return;
  const int Cc = 2 * G * D + H * V;
  const int i = t - cu_q[b];
  const float* held = conv_state + (size_t)slots[b] * (taps - 1) * Cc;
  for (int c = threadIdx.x; c < Cc; c += blockDim.x) {
    float acc = 0.f;
    for (int l = taps - 1; l >= 0; --l) {          // oldest input first
      const int src = i - l;
      const float in = src >= 0 ? x[(size_t)(t - l) * ld + c] : held[(size_t)(taps - 1 + src) * Cc + c];
      acc += taps_w[(size_t)c * taps + (taps - 1 - l)] * in;
    }
    cv[c] = silu_f(acc);
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
  float* o = qkv + (size_t)t * Cc;
  for (int head = warp; head < 2 * G; head += n_warps) {
    const float* hv = cv + (size_t)head * D;
    float ss = 0.f;
    for (int d = lane; d < D; d += 32) ss += hv[d] * hv[d];
    ss = warp_sum(ss);
    const float f = (head < G ? qscale : 1.0f) / sqrtf(ss + unit_eps);
    for (int d = lane; d < D; d += 32) o[(size_t)head * D + d] = hv[d] * f;
  }
  for (int c = 2 * G * D + threadIdx.x; c < Cc; c += blockDim.x) o[c] = cv[c];
  const float* row = x + (size_t)t * ld;
  for (int h = threadIdx.x; h < H; h += blockDim.x) {
    beta[(size_t)t * H + h] = sigmoid_f(row[b_off + h]);
    decay[(size_t)t * H + h] = expf(-expf(A_log[h]) * softplus_f(row[a_off + h] + dt_bias[h]));
  }
}

// conv_state[slot] <- the last taps - 1 inputs of the sequence: a thread per (sequence, channel) reads what it keeps
// of the old rows before it writes.
__global__ void conv_state_update_kernel(const float* __restrict__ x, int ld, float* __restrict__ conv_state, int taps,
                                         const int* __restrict__ cu_q, const int* __restrict__ slots, int n_seqs, int Cc) {
  pdl_wait();
  pdl_trigger();
  const long long id = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (id >= (long long)n_seqs * Cc) return;
  const int b = (int)(id / Cc), c = (int)(id - (long long)b * Cc);
  const int slot = slots[b];
  if (slot < 0) return;
  const int t0 = cu_q[b], n = cu_q[b + 1] - t0, keep = taps - 1;
  float* held = conv_state + (size_t)slot * keep * Cc + c;
  float now[CONV_MAX_TAPS];
#pragma unroll
  for (int s = 0; s < CONV_MAX_TAPS; ++s)
    if (s < keep) {
      const int i = n - keep + s;
      now[s] = i >= 0 ? x[(size_t)(t0 + i) * ld + c] : held[(size_t)(s + n) * Cc];
    }
#pragma unroll
  for (int s = 0; s < CONV_MAX_TAPS; ++s)
    if (s < keep) held[(size_t)s * Cc] = now[s];
}

AB_API int ab_gdr_prepare(const float* x, int ld, const float* taps_w, int taps, float* conv_state, const float* A_log,
                          const float* dt_bias, int b_off, int a_off, float qscale, float unit_eps, float* qkv, float* beta,
                          float* decay, const int* tok_seq, const int* cu_q, const int* slots, int n_tokens, int n_seqs,
                          int H, int G, int D, int V, int write_state, cudaStream_t stream) {
  if (n_tokens <= 0) return AB_OK;
  const int Cc = 2 * G * D + H * V;
  if (taps < 1 || taps > CONV_MAX_TAPS + 1 || H <= 0 || G <= 0 || D <= 0 || V <= 0 || (size_t)Cc * 4 > 200 * 1024) return AB_BAD_ARG;
  if (!x || !taps_w || !conv_state || !A_log || !dt_bias || !qkv || !beta || !decay) return AB_BAD_ARG;
  const size_t smem = (size_t)Cc * sizeof(float);
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(gdr_prepare_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  ab_launch(gdr_prepare_kernel, dim3((unsigned)n_tokens), dim3(256), smem, stream, x, ld, taps_w, taps,
            (const float*)conv_state, A_log, dt_bias, b_off, a_off, qscale, unit_eps, qkv, beta, decay, tok_seq, cu_q, slots,
            H, G, D, V);
  int rc = ab_launch_status();
  if (rc || !write_state || taps == 1) return rc;
  const long long total = (long long)n_seqs * Cc;
  ab_launch(conv_state_update_kernel, dim3((unsigned)((total + 127) / 128)), dim3(128), 0, stream, x, ld, conv_state, taps,
            cu_q, slots, n_seqs, Cc);
  return ab_launch_status();
}

// out[t, h, j] = cast(o[t, h, j] / sqrt(mean_j(o[t, h, :]^2) + eps) * w[j] * act(g[t * ldg + h * V + j]));
// act: 0 none, 1 SiLU, 2 sigmoid.  A warp per (token, head).
template <typename TO>
__global__ void head_norm_gate_kernel(const float* __restrict__ o, const float* __restrict__ w, const float* __restrict__ g,
                                      int ldg, int act, TO* __restrict__ out, const int* __restrict__ tok_seq,
                                      int n_tokens, int H, int V, float eps) {
  pdl_wait();
  pdl_trigger();
  const int lane = threadIdx.x & 31;
  const long long id = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (id >= (long long)n_tokens * H) return;
  const int t = (int)(id / H), h = (int)(id - (long long)t * H);
  TO* dst = out + ((size_t)t * H + h) * V;
  if (tok_seq != nullptr && tok_seq[t] < 0) {
    for (int j = lane; j < V; j += 32) dst[j] = from_f32<TO>(0.f);
    return;
  }
  const float* src = o + ((size_t)t * H + h) * V;
  float ss = 0.f;
  for (int j = lane; j < V; j += 32) ss += src[j] * src[j];
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / (float)V + eps);
  const float* gr = g != nullptr ? g + (size_t)t * ldg + (size_t)h * V : nullptr;
  for (int j = lane; j < V; j += 32) {
    float y = src[j] * inv * (w != nullptr ? w[j] : 1.0f);
    if (gr != nullptr) y *= act == 1 ? silu_f(gr[j]) : (act == 2 ? sigmoid_f(gr[j]) : gr[j]);
    dst[j] = from_f32<TO>(y);
  }
}

AB_API int ab_head_norm_gate(const float* o, const float* w, const float* g, int ldg, int act, void* out, int out_dtype,
                             const int* tok_seq, int n_tokens, int H, int V, float eps, cudaStream_t stream) {
  if (n_tokens <= 0) return AB_OK;
  if (!o || !out || H <= 0 || V <= 0 || act < 0 || act > 2) return AB_BAD_ARG;
  const long long warps = (long long)n_tokens * H;
  const unsigned blocks = (unsigned)((warps + 7) / 8);
  if (out_dtype == AB_F32)
    ab_launch(head_norm_gate_kernel<float>, dim3(blocks), dim3(256), 0, stream, o, w, g, ldg, act, (float*)out, tok_seq,
              n_tokens, H, V, eps);
  else if (out_dtype == AB_BF16)
    ab_launch(head_norm_gate_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, o, w, g, ldg, act, (bf16*)out, tok_seq,
              n_tokens, H, V, eps);
  else
    return AB_BAD_ARG;
  return ab_launch_status();
}
