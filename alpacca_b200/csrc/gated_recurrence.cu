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
// over four neighbouring lanes' registers (rows r, r + 4, ..), q, k and the decays of eight tokens at a time wait in
// shared memory, a column's dot products are summed over its four lanes by shuffles.  The order of additions depends
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
#define CONV_MAX_TAPS 16

__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + expf(-x)); }

template <int DR, int MODE>
__global__ void recurrence_kernel(const float* __restrict__ q, int ldq, const float* __restrict__ k, int ldk,
                                  const float* __restrict__ v, int ldv, const float* __restrict__ dvec, int ldd,
                                  const float* __restrict__ dsc, const float* __restrict__ beta, float qscale,
                                  float* __restrict__ state, float* __restrict__ out, const int* __restrict__ cu_q,
                                  const int* __restrict__ slots, int H, int Hk, int D, int V, int CV, int write_state) {
  extern __shared__ float rec_sm[];
  constexpr int D4 = DR * 4;
  pdl_wait();
  pdl_trigger();
  const int b = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * CV;
  const int slot = slots[b];
  if (slot < 0) return;
  const int kh = h / (H / Hk);
  const int tid = threadIdx.x, col = tid >> 2, r = tid & 3;
  const int j = col0 + col;
  float* qs = rec_sm;                          // [REC_TOKENS][D4]
  float* ks = qs + REC_TOKENS * D4;            // [REC_TOKENS][D4]
  float* as = ks + REC_TOKENS * D4;            // [REC_TOKENS][D4]   (mode 0)
  float* vs = as + (MODE == 0 ? REC_TOKENS * D4 : 0);      // [REC_TOKENS][CV]
  float* os = vs + REC_TOKENS * CV;            // [REC_TOKENS][CV]
  float* sc = os + REC_TOKENS * CV;            // [REC_TOKENS][2]    (mode 1: g, beta)
  float S[DR];
  float* st = state + ((size_t)slot * H + h) * D * V;
#pragma unroll
  for (int i = 0; i < DR; ++i) {
    const int d = r + 4 * i;
    S[i] = (d < D && j < V) ? st[(size_t)d * V + j] : 0.f;
  }
  const int t0 = cu_q[b], t1 = cu_q[b + 1];
  for (int c0 = t0; c0 < t1; c0 += REC_TOKENS) {
    const int n = min(REC_TOKENS, t1 - c0);
    __syncthreads();
    for (int idx = tid; idx < n * D4; idx += blockDim.x) {
      const int tt = idx / D4, d = idx - tt * D4;
      const size_t t = (size_t)(c0 + tt);
      const bool in = d < D;
      qs[idx] = in ? q[t * ldq + (size_t)kh * D + d] * qscale : 0.f;
      ks[idx] = in ? k[t * ldk + (size_t)kh * D + d] : 0.f;
      if (MODE == 0) as[idx] = in ? dvec[t * ldd + (size_t)h * D + d] : 0.f;
    }
    for (int idx = tid; idx < n * CV; idx += blockDim.x) {
      const int tt = idx / CV, c = idx - tt * CV;
      vs[idx] = col0 + c < V ? v[(size_t)(c0 + tt) * ldv + (size_t)h * V + col0 + c] : 0.f;
    }
    if (MODE == 1)
      for (int idx = tid; idx < n; idx += blockDim.x) {
        sc[2 * idx] = dsc[(size_t)(c0 + idx) * H + h];
        sc[2 * idx + 1] = beta[(size_t)(c0 + idx) * H + h];
      }
    __syncthreads();
    for (int tt = 0; tt < n; ++tt) {
      const float vj = vs[tt * CV + col];
      const float* qr = qs + tt * D4 + r;
      const float* kr = ks + tt * D4 + r;
      float acc = 0.f;
      if (MODE == 0) {
        const float* ar = as + tt * D4 + r;
#pragma unroll
        for (int i = 0; i < DR; ++i) {
          S[i] = ar[4 * i] * S[i] + kr[4 * i] * vj;
          acc += S[i] * qr[4 * i];
        }
      } else {
        const float g = sc[2 * tt], bt = sc[2 * tt + 1];
        float dot = 0.f;
#pragma unroll
        for (int i = 0; i < DR; ++i) {
          S[i] *= g;
          dot += S[i] * kr[4 * i];
        }
        dot += __shfl_xor_sync(0xffffffffu, dot, 1);
        dot += __shfl_xor_sync(0xffffffffu, dot, 2);
        const float u = bt * (vj - dot);
#pragma unroll
        for (int i = 0; i < DR; ++i) {
          S[i] += kr[4 * i] * u;
          acc += S[i] * qr[4 * i];
        }
      }
      acc += __shfl_xor_sync(0xffffffffu, acc, 1);
      acc += __shfl_xor_sync(0xffffffffu, acc, 2);
      if (r == 0) os[tt * CV + col] = acc;
    }
    __syncthreads();
    for (int idx = tid; idx < n * CV; idx += blockDim.x) {
      const int tt = idx / CV, c = idx - tt * CV;
      if (col0 + c < V) out[(size_t)(c0 + tt) * H * V + (size_t)h * V + col0 + c] = os[idx];
    }
  }
  if (!write_state) return;
#pragma unroll
  for (int i = 0; i < DR; ++i) {
    const int d = r + 4 * i;
    if (d < D && j < V) st[(size_t)d * V + j] = S[i];
  }
}

// One walk over the step's tokens.  q, k float32 rows with Hk heads of D (row strides ldq, ldk), v with H heads of V;
// mode 0: dvec [T, H * D] (row stride ldd); mode 1: dsc, beta [T, H].  state [slots, H, D, V]; out [T, H * V].
// `cols`: value columns per CTA (8, 16 or 32).
AB_API int ab_gated_recurrence(int mode, const float* q, int ldq, const float* k, int ldk, const float* v, int ldv,
                               const float* dvec, int ldd, const float* dsc, const float* beta, float qscale, float* state,
                               float* out, const int* cu_q, const int* slots, int n_seqs, int H, int Hk, int D, int V,
                               int cols, int write_state, cudaStream_t stream) {
  if (n_seqs <= 0) return AB_OK;
  if (H <= 0 || Hk <= 0 || H % Hk || D <= 0 || D > 256 || V <= 0 || (cols != 8 && cols != 16 && cols != 32)) return AB_BAD_ARG;
  if (!q || !k || !v || !state || !out || !cu_q || !slots) return AB_BAD_ARG;
  if (mode == 0 ? !dvec : (mode != 1 || !dsc || !beta)) return AB_BAD_ARG;
  const int DR = D <= 32 ? 8 : (D <= 64 ? 16 : (D <= 128 ? 32 : 64));
  const int D4 = DR * 4;
  const size_t smem = sizeof(float) * ((size_t)REC_TOKENS * D4 * (mode == 0 ? 3 : 2) + 2 * REC_TOKENS * cols + 2 * REC_TOKENS);
  const dim3 grid((unsigned)n_seqs, (unsigned)H, (unsigned)((V + cols - 1) / cols));
  const dim3 block((unsigned)cols * 4);
#define AB_GO(DRV, M)                                                                                                \
  ab_launch(recurrence_kernel<DRV, M>, grid, block, smem, stream, q, ldq, k, ldk, v, ldv, dvec, ldd, dsc, beta, qscale, \
            state, out, cu_q, slots, H, Hk, D, V, cols, write_state)
  if (mode == 0) {
    if (DR == 8) AB_GO(8, 0); else if (DR == 16) AB_GO(16, 0); else if (DR == 32) AB_GO(32, 0); else AB_GO(64, 0);
  } else {
    if (DR == 8) AB_GO(8, 1); else if (DR == 16) AB_GO(16, 1); else if (DR == 32) AB_GO(32, 1); else AB_GO(64, 1);
  }
#undef AB_GO
  return ab_launch_status();
}

// a[t, c] = sigmoid(z)^(1/tau), z = b[c] + sum_r W2[c, r] y[t, r]; y: `rank` numbers per token at y + t * ldy.
// A block of 128 channels x 8 tokens, so a row of W2 is read once for eight tokens.
__global__ void gla_decay_kernel(const float* __restrict__ y, int ldy, const float* __restrict__ w2,
                                 const float* __restrict__ bias, float inv_tau, float* __restrict__ a, int n_tokens,
                                 int channels, int rank) {
  extern __shared__ float ys[];              // [8][rank]
  pdl_wait();
  pdl_trigger();
  const int t0 = blockIdx.y * 8, n = min(8, n_tokens - t0);
  for (int idx = threadIdx.x; idx < n * rank; idx += blockDim.x) {
    const int tt = idx / rank, rr = idx - tt * rank;
    ys[idx] = y[(size_t)(t0 + tt) * ldy + rr];
  }
  __syncthreads();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  float z[8];
  const float bc = bias != nullptr ? bias[c] : 0.f;
#pragma unroll
  for (int tt = 0; tt < 8; ++tt) z[tt] = bc;
  const float* wr = w2 + (size_t)c * rank;
  for (int rr = 0; rr < rank; ++rr) {
    const float w = wr[rr];
#pragma unroll
    for (int tt = 0; tt < 8; ++tt)
      if (tt < n) z[tt] += w * ys[tt * rank + rr];
  }
#pragma unroll
  for (int tt = 0; tt < 8; ++tt)
    if (tt < n) a[(size_t)(t0 + tt) * channels + c] = expf(-softplus_f(-z[tt]) * inv_tau);     // log sigmoid(z) = -softplus(-z)
}

AB_API int ab_gla_decay(const float* y, int ldy, const float* w2, const float* bias, float tau, float* a, int n_tokens,
                        int channels, int rank, cudaStream_t stream) {
  if (n_tokens <= 0) return AB_OK;
  if (!y || !w2 || !a || channels <= 0 || rank <= 0 || !(tau > 0.f) || (size_t)rank * 32 > 48 * 1024) return AB_BAD_ARG;
  const dim3 grid((unsigned)((channels + 127) / 128), (unsigned)((n_tokens + 7) / 8));
  ab_launch(gla_decay_kernel, grid, dim3(128), (size_t)8 * rank * sizeof(float), stream, y, ldy, w2, bias, 1.0f / tau, a,
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
