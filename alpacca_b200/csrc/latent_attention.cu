// Attention over a cached latent: every head reads the same row per position, [c (C dims) | r (R dims)],
// where c is the normed low-rank latent of keys and values and r one rotated key part for all heads.
// With the keys' up-projection folded into the query (q' = W_uk_h^T q_unrotated, C dims) the score of head
// h at key s is (q'_h . c_s + q_rot_h . r_s) * scale, and the head's output is W_uv_h (sum_s p_s c_s): the
// cache is never expanded.  The softmax's denominator also holds exp(sink_h), which has no key and no value.
//
// Kernels (32-bit arithmetic; storage float or bfloat16):
//   latent_prep     per token: RMS norm of the query latent, RMS norm of c, rotation of r by position, and
//                   the append of [c | r] to the sequence's page;
//   heads_matmul    out[t, h, n] = sum_k a[t, h, k] w[h, n, k], one warp per output; with a tail of
//                   rotated dims copied behind it (the query's rotated part);
//   latent_attention_simt   one warp per (token, head) walks the keys in order (online softmax).
#include "common.cuh"
#include "launch.cuh"

// ---------------------------------------------------------------------------------------------
// x: [T, ld] float32 = q latent (Q dims) | c (C dims) | r (R dims).  One block per token.
template <typename TA>
__global__ void latent_prep_kernel(const float* __restrict__ x, int ld, int Q, int C, int R,
                                   const float* __restrict__ wq, const float* __restrict__ wc, float eps,
                                   const float* __restrict__ cos_t, const float* __restrict__ sin_t, int n_rot,
                                   const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                                   const int* __restrict__ block_table, int table_width, int page_size,
                                   TA* __restrict__ pages, TA* __restrict__ cq_out, int write_cache) {
  __shared__ float scratch[32];
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  const int b = tok_seq[t];
  if (b < 0) return;
  const float* row = x + (size_t)t * ld;
  float ss = 0.f;
  for (int j = threadIdx.x; j < Q; j += blockDim.x) ss += row[j] * row[j];
  ss = block_sum(ss, scratch);
  const float inv_q = 1.0f / sqrtf(ss / (float)Q + eps);
  for (int j = threadIdx.x; j < Q; j += blockDim.x) cq_out[(size_t)t * Q + j] = from_f32<TA>(row[j] * inv_q * wq[j]);
  if (!write_cache) return;
  const float* c = row + Q;
  ss = 0.f;
  for (int j = threadIdx.x; j < C; j += blockDim.x) ss += c[j] * c[j];
  ss = block_sum(ss, scratch);
  const float inv_c = 1.0f / sqrtf(ss / (float)C + eps);
  const int pos = tok_pos[t];
  const int page = block_table[(size_t)b * table_width + pos / page_size];
  TA* dst = pages + ((size_t)page * page_size + (pos % page_size)) * (C + R);
  for (int j = threadIdx.x; j < C; j += blockDim.x) dst[j] = from_f32<TA>(c[j] * inv_c * wc[j]);
  const float* r = c + C;
  const int half = n_rot / 2;
  for (int j = threadIdx.x; j < R; j += blockDim.x) {
    float v = r[j];
    if (j < n_rot) {
      const int i = j >> 1;
      const float cs = cos_t[(size_t)pos * half + i], sn = sin_t[(size_t)pos * half + i];
      v = (j & 1) ? r[j] * cs + r[j - 1] * sn : r[j] * cs - r[j + 1] * sn;
    }
    dst[C + j] = from_f32<TA>(v);
  }
}

AB_API int ab_latent_prep(const float* x, int ld, int Q, int C, int R, const float* wq, const float* wc, float eps,
                          const float* cos_t, const float* sin_t, int n_rot, const int* tok_pos, const int* tok_seq,
                          const int* block_table, int table_width, int page_size, void* pages, void* cq_out,
                          int dtype, int n_tokens, int write_cache, cudaStream_t stream) {
  if (n_tokens <= 0) return AB_OK;
  // a caller that writes no cache (a layer that reads another layer's latent) gives rows of the Q numbers alone
  if (Q <= 0 || C <= 0 || R < 0 || n_rot < 0 || n_rot > R || (n_rot & 1) || ld < (write_cache ? Q + C + R : Q)) return AB_BAD_ARG;
  if (dtype == AB_F32)
    ab_launch(latent_prep_kernel<float>, dim3(n_tokens), dim3(128), 0, stream, x, ld, Q, C, R, wq, wc, eps, cos_t, sin_t,
              n_rot, tok_pos, tok_seq, block_table, table_width, page_size, (float*)pages, (float*)cq_out, write_cache);
  else if (dtype == AB_BF16)
    ab_launch(latent_prep_kernel<bf16>, dim3(n_tokens), dim3(128), 0, stream, x, ld, Q, C, R, wq, wc, eps, cos_t, sin_t,
              n_rot, tok_pos, tok_seq, block_table, table_width, page_size, (bf16*)pages, (bf16*)cq_out, write_cache);
  else
    return AB_BAD_ARG;
  return ab_launch_status();
}

// ---------------------------------------------------------------------------------------------
// a: [T, H, a_hs] (row stride lda), w: [H, N, K], out: [T, H, o_hs] (row stride ldo).  Warp per (t, h, n).
// tail > 0: out[t, h, tail_at + j] = a[t, h, K + j] for j < tail, its first n_rot dims rotated in pairs (2i, 2i+1).
template <typename TA, typename TW, typename TO>
__global__ void heads_matmul_kernel(const TA* __restrict__ a, int lda, int a_hs, const TW* __restrict__ w,
                                    TO* __restrict__ out, int ldo, int o_hs, int n_tokens, int H, int N, int K,
                                    int tail, int tail_at, const float* __restrict__ cos_t,
                                    const float* __restrict__ sin_t, int n_rot, const int* __restrict__ tok_pos,
                                    const int* __restrict__ tok_seq) {
  pdl_wait();
  pdl_trigger();
  const int lane = threadIdx.x & 31;
  const int per = N + tail;
  const long long id = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (id >= (long long)n_tokens * H * per) return;
  const int n = (int)(id % per);
  const long long th = id / per;
  const int h = (int)(th % H), t = (int)(th / H);
  if (tok_seq != nullptr && tok_seq[t] < 0) return;
  const TA* av = a + (size_t)t * lda + (size_t)h * a_hs;
  TO* o = out + (size_t)t * ldo + (size_t)h * o_hs;
  if (n < N) {
    const TW* wr = w + ((size_t)h * N + n) * K;
    float part = 0.f;
    for (int k = lane; k < K; k += 32) part += to_f32(av[k]) * to_f32(wr[k]);
    part = warp_sum(part);
    if (lane == 0) o[n] = from_f32<TO>(part);
    return;
  }
  if (lane != 0) return;
  const int j = n - N;
  float v = to_f32(av[K + j]);
  if (j < n_rot) {
    const int pos = tok_pos[t], half = n_rot / 2, i = j >> 1;
    const float cs = cos_t[(size_t)pos * half + i], sn = sin_t[(size_t)pos * half + i];
    v = (j & 1) ? v * cs + to_f32(av[K + j - 1]) * sn : v * cs - to_f32(av[K + j + 1]) * sn;
  }
  o[tail_at + j] = from_f32<TO>(v);
}

template <typename TA, typename TW, typename TO>
static int heads_go(const void* a, int lda, int a_hs, const void* w, void* out, int ldo, int o_hs, int n_tokens, int H,
                    int N, int K, int tail, int tail_at, const float* cos_t, const float* sin_t, int n_rot,
                    const int* tok_pos, const int* tok_seq, cudaStream_t stream) {
  const long long warps = (long long)n_tokens * H * (N + tail);
  const int wpb = 8;
  const long long blocks = (warps + wpb - 1) / wpb;
  if (blocks > 0x7fffffffLL) return AB_BAD_ARG;
  ab_launch(heads_matmul_kernel<TA, TW, TO>, dim3((unsigned)blocks), dim3(wpb * 32), 0, stream, (const TA*)a, lda, a_hs,
            (const TW*)w, (TO*)out, ldo, o_hs, n_tokens, H, N, K, tail, tail_at, cos_t, sin_t, n_rot, tok_pos, tok_seq);
  return ab_launch_status();
}

// dtypes: a, w, out each AB_F32 or AB_BF16; supported: (f32,f32,f32), (bf16,bf16,f32), (bf16,bf16,bf16), (f32,bf16,bf16),
// (f32,bf16,f32)
AB_API int ab_heads_matmul(const void* a, int a_dt, int lda, int a_hs, const void* w, int w_dt, void* out, int o_dt,
                           int ldo, int o_hs, int n_tokens, int H, int N, int K, int tail, int tail_at,
                           const float* cos_t, const float* sin_t, int n_rot, const int* tok_pos, const int* tok_seq,
                           cudaStream_t stream) {
  if (n_tokens <= 0) return AB_OK;
  if (H <= 0 || N < 0 || N + tail <= 0 || K <= 0 || tail < 0 || n_rot > tail || (n_rot & 1) || tail_at < N ||
      tail_at + tail > o_hs)
    return AB_BAD_ARG;
#define AB_HM(TA, TW, TO)                                                                                        \
  return heads_go<TA, TW, TO>(a, lda, a_hs, w, out, ldo, o_hs, n_tokens, H, N, K, tail, tail_at, cos_t, sin_t, n_rot, \
                              tok_pos, tok_seq, stream)
  if (a_dt == AB_F32 && w_dt == AB_F32 && o_dt == AB_F32) AB_HM(float, float, float);
  if (a_dt == AB_BF16 && w_dt == AB_BF16 && o_dt == AB_F32) AB_HM(bf16, bf16, float);
  if (a_dt == AB_BF16 && w_dt == AB_BF16 && o_dt == AB_BF16) AB_HM(bf16, bf16, bf16);
  if (a_dt == AB_F32 && w_dt == AB_BF16 && o_dt == AB_BF16) AB_HM(float, bf16, bf16);
  if (a_dt == AB_F32 && w_dt == AB_BF16 && o_dt == AB_F32) AB_HM(float, bf16, float);
  if (a_dt == AB_BF16 && w_dt == AB_F32 && o_dt == AB_BF16) AB_HM(bf16, float, bf16);
#undef AB_HM
  return AB_BAD_ARG;
}

// ---------------------------------------------------------------------------------------------
// q: [T, H, C + R] float32; pages: [n_pages, page, C + R]; out: [T, H, C] float32.  One warp per (token, head);
// lane l owns dims l, l + 32, ...  The keys are walked in order, so a token's result does not depend on the
// rest of the batch or on how the prompt was cut.
template <typename TC, int DPL>
__global__ void latent_attention_simt_kernel(const float* __restrict__ q, float* __restrict__ out,
                                             const TC* __restrict__ pages, const int* __restrict__ block_table,
                                             int table_width, const int* __restrict__ tok_pos,
                                             const int* __restrict__ tok_seq, const float* __restrict__ sink,
                                             int n_tokens, int H, int C, int R, int page_size, float scale,
                                             int window) {
  pdl_wait();
  pdl_trigger();
  const int lane = threadIdx.x & 31;
  const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (w >= (long long)n_tokens * H) return;
  const int t = (int)(w / H), h = (int)(w - (long long)t * H);
  const int b = tok_seq[t];
  if (b < 0) return;
  const int Dk = C + R;
  const int pos = tok_pos[t];
  const float* qv = q + ((size_t)t * H + h) * Dk;
  float qr[DPL], acc[DPL];
#pragma unroll
  for (int j = 0; j < DPL; ++j) {
    const int d = lane + 32 * j;
    qr[j] = d < Dk ? qv[d] * scale : 0.f;
    acc[j] = 0.f;
  }
  float m = -INFINITY, l = 0.f;
  const int* bt = block_table + (size_t)b * table_width;
  for (int s = window > 0 ? max(0, pos - window + 1) : 0; s <= pos; ++s) {
    const int page = bt[s / page_size];
    const TC* kv = pages + ((size_t)page * page_size + (s % page_size)) * Dk;
    float kr[DPL];
    float part = 0.f;
#pragma unroll
    for (int j = 0; j < DPL; ++j) {
      const int d = lane + 32 * j;
      kr[j] = d < Dk ? to_f32(kv[d]) : 0.f;
      part += qr[j] * kr[j];
    }
    const float score = warp_sum(part);
    const float m_new = fmaxf(m, score);
    const float corr = expf(m - m_new);
    const float p = expf(score - m_new);
    l = l * corr + p;
#pragma unroll
    for (int j = 0; j < DPL; ++j) acc[j] = acc[j] * corr + p * kr[j];
    m = m_new;
  }
  // the sink: one more term of the denominator, without a value
  const float sk = sink != nullptr ? sink[h] : -INFINITY;
  const float m_all = fmaxf(m, sk);
  const float corr = expf(m - m_all);
  l = l * corr + (sink != nullptr ? expf(sk - m_all) : 0.f);
  const float inv = corr / l;
  float* o = out + ((size_t)t * H + h) * C;
#pragma unroll
  for (int j = 0; j < DPL; ++j) {
    const int d = lane + 32 * j;
    if (d < C) o[d] = acc[j] * inv;
  }
}

template <typename TC>
static int latent_simt_go(const float* q, float* out, const void* pages, const int* block_table, int table_width,
                          const int* tok_pos, const int* tok_seq, const float* sink, int n_tokens, int H, int C, int R,
                          int page_size, float scale, int window, cudaStream_t stream) {
  const long long warps = (long long)n_tokens * H;
  const int wpb = 4;
  const unsigned blocks = (unsigned)((warps + wpb - 1) / wpb);
  const int dpl = (C + R + 31) / 32;
#define AB_GO(DPL)                                                                                                \
  latent_attention_simt_kernel<TC, DPL><<<blocks, wpb * 32, 0, stream>>>(q, out, (const TC*)pages, block_table,   \
                                                                         table_width, tok_pos, tok_seq, sink,    \
                                                                         n_tokens, H, C, R, page_size, scale, window)
  if (dpl <= 1) AB_GO(1);
  else if (dpl <= 2) AB_GO(2);
  else if (dpl <= 4) AB_GO(4);
  else if (dpl <= 8) AB_GO(8);
  else if (dpl <= 12) AB_GO(12);
  else if (dpl <= 18) AB_GO(18);
  else AB_GO(32);
#undef AB_GO
  return ab_launch_status();
}

// `window` > 0: a token sees itself and the window - 1 tokens before it
AB_API int ab_latent_attention_simt_window(const float* q, float* out, const void* pages, int dtype,
                                           const int* block_table, int table_width, const int* tok_pos,
                                           const int* tok_seq, const float* sink, int n_tokens, int H, int C, int R,
                                           int page_size, float scale, int window, cudaStream_t stream) {
  if (n_tokens <= 0) return AB_OK;
  if (H <= 0 || C <= 0 || R < 0 || C + R > 1024 || window < 0) return AB_BAD_ARG;
  if (dtype == AB_F32)
    return latent_simt_go<float>(q, out, pages, block_table, table_width, tok_pos, tok_seq, sink, n_tokens, H, C, R,
                                 page_size, scale, window, stream);
  if (dtype == AB_BF16)
    return latent_simt_go<bf16>(q, out, pages, block_table, table_width, tok_pos, tok_seq, sink, n_tokens, H, C, R,
                                page_size, scale, window, stream);
  return AB_BAD_ARG;
}

AB_API int ab_latent_attention_simt(const float* q, float* out, const void* pages, int dtype, const int* block_table,
                                    int table_width, const int* tok_pos, const int* tok_seq, const float* sink,
                                    int n_tokens, int H, int C, int R, int page_size, float scale,
                                    cudaStream_t stream) {
  return ab_latent_attention_simt_window(q, out, pages, dtype, block_table, table_width, tok_pos, tok_seq, sink, n_tokens,
                                         H, C, R, page_size, scale, 0, stream);
}
