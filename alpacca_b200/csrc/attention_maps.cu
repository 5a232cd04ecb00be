// Grouped-query attention over the paged cache whose keys and values have sizes and head counts of their
// own, with one or several score maps per head, 32-bit arithmetic.  Two kernels:
//
//   prepare   one warp per (token, vector): a query vector is (optionally) divided by its root mean square and
//             multiplied by a weight, then rotated by position, in place; a key vector likewise, and written to
//             the key pages; a value vector is copied to the value pages as it was projected.  The values may be
//             read from the same place as the keys (values that are the keys before norm and rotation).
//   attend    one warp per (token, head).  A head has M maps; map m of head h has the query vector h*M + m
//             and reads key head (h / (H/G)) * M + m and value head h / (H/G):
//               a_m = softmax_s((q_m . k_m,s) * scale) v_s   over lo <= s <= p, lo = max(0, p - window + 1)
//             (window 0: all), with exp(sink_h) as one more term of the denominator when sinks are given;
//               o = a_0 + sum_{m>0} coef * a_m,
//             then, if asked, o is divided by its root mean square (eps inside the root), and multiplied by
//             out_scale.  The softmax is the running form, in key order; nothing is shared between warps, so
//             a token's result does not depend on the rest of the batch.
//
//   combine   the last step of `attend` alone, for maps that another kernel has attended (float [T, H*M, Dv]).
//
// Mixing of the softmax weights across heads (Shazeer et al., "Talking-Heads Attention", mix the weights of all heads
// after the softmax):  w'_h(t, s) = sum_g T[h, g] w_g(t, s), and head h applies w'_h to the values of its own
// key/value head c(h).  Since the mixing is linear and every w_g is normalised by itself,
//     o_h = sum_g T[h, g] A[g, c(h)],    A[g, c] = sum_s w_g(t, s) v_c(s),
// so the attention of head g over the values of ALL key/value heads is computed once (the values of a token's heads
// lie side by side in one row of G*Dv numbers: value pages [n_pages, 1, page, G*Dv]) and the mixing is a small
// product afterwards.  The query vectors are then ordered so that vector x reads key head x % G (the order of the
// general tensor-core kernel with G maps in one group): head g = (x % G) * (H/G) + x / G.
//   talk_attend   one warp per (token, query vector x): A[t, x, :] in float32, running softmax in key order
//   talk_combine  one warp per (token, head h): o_h from A and T, times sigmoid of a gate (optional)
//
// `prepare` can divide every value vector by its root mean square (no weight) before it is stored, and can store
// the value heads side by side.
//
// Key pages [n_pages, G*M, page, Dk], value pages [n_pages, G, page, Dv]; one block table for both.
// Rotation: the first n_rot dims of a vector, pairing 0 = (2i, 2i+1), 1 = (i, i + n_rot/2); tables
// float32 [positions, n_rot/2].  (u, v) -> (u cos - v sin, v cos + u sin).
#include "common.cuh"
#include "launch.cuh"

#define AM_MAX_DIM 256

struct PrepareArgs {
  void* buf;               // [T, stride] projected rows; query vectors are rewritten in place
  int stride, off_q, off_k, off_v;
  int n_q, n_k, n_v;       // vectors per token: H*M queries, G*M keys, G values
  int Dk, Dv;
  const float* q_weight;   // [Dk] or null: no norm
  const float* k_weight;
  float eps;
  const float* cos_t; const float* sin_t; int n_rot, pairing;
  const int* tok_pos; const int* tok_seq;
  const int* block_table; int table_width;
  void* k_pages; void* v_pages; int page_size;
  int n_tokens, write_cache;
  const float* bias;       // [stride] or null: added to the projected values first (a projection that left it out)
  int v_norm;              // 1: a value vector is divided by its root mean square (eps inside the root) before it is stored
  int v_side_by_side;      // 1: value pages [n_pages, 1, page, n_v * Dv]: a token's value heads in one row
};

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

template <typename T>
__global__ void __launch_bounds__(128)
attention_prepare_kernel(PrepareArgs a) {
  __shared__ float stage[4][AM_MAX_DIM];
  pdl_wait();
  pdl_trigger();
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  const int per_tok = a.n_q + a.n_k + a.n_v;
  const long long w = (long long)blockIdx.x * 4 + wib;
  if (w >= (long long)a.n_tokens * per_tok) return;
  const int t = (int)(w / per_tok), vec = (int)(w - (long long)t * per_tok);
  const int b = a.tok_seq[t];
  if (b < 0) return;
  const int pos = a.tok_pos[t];
  T* row = reinterpret_cast<T*>(a.buf) + (size_t)t * a.stride;
  const int page = a.write_cache ? a.block_table[(size_t)b * a.table_width + pos / a.page_size] : 0;
  const int in_page = pos % a.page_size;
  if (vec >= a.n_q + a.n_k) {                       // a value vector: copied as projected
    if (!a.write_cache) return;
    const int g = vec - a.n_q - a.n_k;
    const int col = a.off_v + g * a.Dv;
    const T* src = row + col;
    T* dst = a.v_side_by_side
                 ? reinterpret_cast<T*>(a.v_pages) + (((size_t)page * a.page_size + in_page) * a.n_v + g) * a.Dv
                 : reinterpret_cast<T*>(a.v_pages) + (((size_t)page * a.n_v + g) * a.page_size + in_page) * a.Dv;
    if (a.v_norm) {
      float ss = 0.f;
      for (int d = lane; d < a.Dv; d += 32) {
        const float v = to_f32(src[d]) + (a.bias != nullptr ? a.bias[col + d] : 0.f);
        ss += v * v;
      }
      const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)a.Dv + a.eps);
      for (int d = lane; d < a.Dv; d += 32)
        dst[d] = from_f32<T>((to_f32(src[d]) + (a.bias != nullptr ? a.bias[col + d] : 0.f)) * inv);
      return;
    }
    if (a.bias == nullptr) {
      for (int d = lane; d < a.Dv; d += 32) dst[d] = src[d];
    } else {
      for (int d = lane; d < a.Dv; d += 32) dst[d] = from_f32<T>(to_f32(src[d]) + a.bias[col + d]);
    }
    return;
  }
  const bool is_q = vec < a.n_q;
  if (!is_q && !a.write_cache) return;
  const int head = is_q ? vec : vec - a.n_q;
  const int D = a.Dk;
  const int col = (is_q ? a.off_q : a.off_k) + head * D;
  T* src = row + col;
  const float* weight = is_q ? a.q_weight : a.k_weight;
  float* x = stage[wib];
  float ss = 0.f;
  for (int d = lane; d < D; d += 32) {
    const float v = to_f32(src[d]) + (a.bias != nullptr ? a.bias[col + d] : 0.f);
    x[d] = v;
    ss += v * v;
  }
  if (weight != nullptr) {
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)D + a.eps);
    for (int d = lane; d < D; d += 32) x[d] = x[d] * inv * weight[d];
  }
  __syncwarp();
  T* dst = is_q ? src
                : reinterpret_cast<T*>(a.k_pages) + (((size_t)page * a.n_k + head) * a.page_size + in_page) * D;
  const int half = a.n_rot >> 1;
  const float* cr = a.cos_t ? a.cos_t + (size_t)pos * half : nullptr;
  const float* sr = a.cos_t ? a.sin_t + (size_t)pos * half : nullptr;
  for (int d = lane; d < D; d += 32) {
    float v = x[d];
    if (cr != nullptr && d < a.n_rot) {
      int i, partner;
      bool first;
      if (a.pairing == 0) { i = d >> 1; first = (d & 1) == 0; partner = d ^ 1; }
      else { first = d < half; i = first ? d : d - half; partner = first ? d + half : d - half; }
      const float p = x[partner], c = cr[i], s = sr[i];
      v = first ? v * c - p * s : v * c + p * s;
    }
    dst[d] = from_f32<T>(v);
  }
}

// The same for bfloat16 rows in 16-byte pieces.  Query and key vectors: a lane owns 8 consecutive elements, a
// vector takes P = Dk / 8 neighbouring lanes, a warp floor(32 / P) vectors (the norm's sum and the partner of a pair
// in the other half come by shuffles inside the vector's lanes).  Value vectors: the warps after those, a lane per
// piece.  Needs Dk, Dv, the offsets and the row stride to be multiples of 8, and for the pairing in halves n_rot a
// multiple of 16 (a pair's two elements then sit at the same place of two pieces).
__global__ void __launch_bounds__(128)
attention_prepare_vec_kernel(PrepareArgs a, int P, int vec_per_warp, long long qk_warps) {
  pdl_wait();
  pdl_trigger();
  const int lane = threadIdx.x & 31;
  const long long warp = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (warp >= qk_warps) {
    // value pieces: copied as projected (plus the bias)
    if (!a.write_cache) return;
    const int Pv = a.Dv >> 3;
    const long long i = (warp - qk_warps) * 32 + lane;
    if (i >= (long long)a.n_tokens * a.n_v * Pv) return;
    const int t = (int)(i / (a.n_v * Pv));
    const int rest = (int)(i - (long long)t * (a.n_v * Pv));
    const int g = rest / Pv, piece = rest - g * Pv;
    const int b = a.tok_seq[t];
    if (b < 0) return;
    const int pos = a.tok_pos[t];
    const int col = a.off_v + g * a.Dv + piece * 8;
    uint4 raw = *reinterpret_cast<const uint4*>(reinterpret_cast<const bf16*>(a.buf) + (size_t)t * a.stride + col);
    if (a.bias != nullptr) {
      const float4 b0 = *reinterpret_cast<const float4*>(a.bias + col), b1 = *reinterpret_cast<const float4*>(a.bias + col + 4);
      raw.x = pack2(__uint_as_float(raw.x << 16) + b0.x, __uint_as_float(raw.x & 0xffff0000u) + b0.y);
      raw.y = pack2(__uint_as_float(raw.y << 16) + b0.z, __uint_as_float(raw.y & 0xffff0000u) + b0.w);
      raw.z = pack2(__uint_as_float(raw.z << 16) + b1.x, __uint_as_float(raw.z & 0xffff0000u) + b1.y);
      raw.w = pack2(__uint_as_float(raw.w << 16) + b1.z, __uint_as_float(raw.w & 0xffff0000u) + b1.w);
    }
    const int page = a.block_table[(size_t)b * a.table_width + pos / a.page_size];
    bf16* dst = a.v_side_by_side
                    ? reinterpret_cast<bf16*>(a.v_pages) +
                          (((size_t)page * a.page_size + pos % a.page_size) * a.n_v + g) * a.Dv + piece * 8
                    : reinterpret_cast<bf16*>(a.v_pages) +
                          (((size_t)page * a.n_v + g) * a.page_size + pos % a.page_size) * a.Dv + piece * 8;
    *reinterpret_cast<uint4*>(dst) = raw;
    return;
  }
  const int per_tok = a.n_q + a.n_k;
  const long long total = (long long)a.n_tokens * per_tok;
  const int vw = lane / P, piece = lane - vw * P;
  const long long w = warp * vec_per_warp + vw;
  const bool live_lane = vw < vec_per_warp && w < total;
  // every lane of a warp walks the same shuffles; lanes without a vector carry zeros
  int t = 0, vec = 0, b = -1, pos = 0;
  if (live_lane) {
    t = (int)(w / per_tok);
    vec = (int)(w - (long long)t * per_tok);
    b = a.tok_seq[t];
    pos = a.tok_pos[t];
  }
  const bool is_q = vec < a.n_q;
  const bool live = live_lane && b >= 0 && (is_q || a.write_cache);
  const int head = is_q ? vec : vec - a.n_q;
  const int D = a.Dk;
  const int col = (is_q ? a.off_q : a.off_k) + head * D + piece * 8;
  bf16* row = reinterpret_cast<bf16*>(a.buf) + (size_t)t * a.stride;
  float x[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) x[j] = 0.f;
  if (live) {
    const uint4 raw = *reinterpret_cast<const uint4*>(row + col);
    const uint32_t wd[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      x[2 * j] = __uint_as_float(wd[j] << 16);
      x[2 * j + 1] = __uint_as_float(wd[j] & 0xffff0000u);
    }
    if (a.bias != nullptr) {
      const float4 b0 = *reinterpret_cast<const float4*>(a.bias + col), b1 = *reinterpret_cast<const float4*>(a.bias + col + 4);
      x[0] += b0.x; x[1] += b0.y; x[2] += b0.z; x[3] += b0.w; x[4] += b1.x; x[5] += b1.y; x[6] += b1.z; x[7] += b1.w;
    }
  }
  const float* weight = is_q ? a.q_weight : a.k_weight;
  if (a.q_weight != nullptr || a.k_weight != nullptr) {   // the same for the whole launch: no lane leaves the shuffles
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += x[j] * x[j];
    float tot = 0.f;
    for (int j = 0; j < P; ++j) tot += __shfl_sync(0xffffffffu, ss, (vw * P + j) & 31);
    if (live && weight != nullptr) {
      const float inv = 1.0f / sqrtf(tot / (float)D + a.eps);
      const float4 w0 = *reinterpret_cast<const float4*>(weight + piece * 8), w1 = *reinterpret_cast<const float4*>(weight + piece * 8 + 4);
      x[0] *= inv * w0.x; x[1] *= inv * w0.y; x[2] *= inv * w0.z; x[3] *= inv * w0.w;
      x[4] *= inv * w1.x; x[5] *= inv * w1.y; x[6] *= inv * w1.z; x[7] *= inv * w1.w;
    }
  }
  if (a.cos_t != nullptr) {
    const int half = a.n_rot >> 1;
    const bool turn = live && piece * 8 < a.n_rot;
    if (a.pairing == 0) {
      if (turn) {
        const float* cr = a.cos_t + (size_t)pos * half + piece * 4;
        const float* sr = a.sin_t + (size_t)pos * half + piece * 4;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (piece * 8 + 2 * j < a.n_rot) {
            const float u = x[2 * j], v = x[2 * j + 1], c = cr[j], sn = sr[j];
            x[2 * j] = u * c - v * sn;
            x[2 * j + 1] = v * c + u * sn;
          }
        }
      }
    } else {
      // halves: the partner piece is half / 8 lanes away, on the other side of the middle
      const int hp = half >> 3;
      const bool first = piece < hp;
      const int partner = (vw * P + (first ? piece + hp : piece - hp)) & 31;
      float p[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) p[j] = __shfl_sync(0xffffffffu, x[j], partner);
      if (turn) {
        const int i0 = (first ? piece : piece - hp) * 8;
        const float* cr = a.cos_t + (size_t)pos * half + i0;
        const float* sr = a.sin_t + (size_t)pos * half + i0;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float c = cr[j], sn = sr[j];
          x[j] = first ? x[j] * c - p[j] * sn : x[j] * c + p[j] * sn;
        }
      }
    }
  }
  if (!live) return;
  uint4 out;
  out.x = pack2(x[0], x[1]); out.y = pack2(x[2], x[3]); out.z = pack2(x[4], x[5]); out.w = pack2(x[6], x[7]);
  if (is_q) {
    *reinterpret_cast<uint4*>(row + col) = out;
    return;
  }
  const int page = a.block_table[(size_t)b * a.table_width + pos / a.page_size];
  bf16* dst = reinterpret_cast<bf16*>(a.k_pages) +
              (((size_t)page * a.n_k + head) * a.page_size + pos % a.page_size) * D + piece * 8;
  *reinterpret_cast<uint4*>(dst) = out;
}

struct AttendArgs {
  const void* q; int q_stride;      // query vectors of token t at q + t*q_stride + (h*M + m)*Dk
  void* out;                        // [T, H*Dv]
  const void* k_pages; const void* v_pages;
  const int* block_table; int table_width;
  const int* tok_pos; const int* tok_seq;
  int n_tokens, H, G, M, Dk, Dv, page_size;
  float scale; int window;
  const float* sink;                // [H] or null
  float coef;                       // weight of every map after the first
  int unit_norm; float eps, out_scale;
};

template <typename T, int KPL, int VPL>
__global__ void __launch_bounds__(128)
attention_maps_kernel(AttendArgs a) {
  pdl_wait();
  pdl_trigger();
  const int lane = threadIdx.x & 31;
  const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (w >= (long long)a.n_tokens * a.H) return;
  const int t = (int)(w / a.H), h = (int)(w - (long long)t * a.H);
  const int Dk = a.Dk, Dv = a.Dv, M = a.M;
  T* o = reinterpret_cast<T*>(a.out) + ((size_t)t * a.H + h) * Dv;
  const int b = a.tok_seq[t];
  if (b < 0) {
    for (int d = lane; d < Dv; d += 32) o[d] = from_f32<T>(0.f);
    return;
  }
  const int pos = a.tok_pos[t];
  const int g = h / (a.H / a.G);
  const int lo = (a.window > 0 && pos - a.window + 1 > 0) ? pos - a.window + 1 : 0;
  const int* bt = a.block_table + (size_t)b * a.table_width;
  const T* kp = reinterpret_cast<const T*>(a.k_pages);
  const T* vp = reinterpret_cast<const T*>(a.v_pages);
  float total[VPL];
#pragma unroll
  for (int j = 0; j < VPL; ++j) total[j] = 0.f;
  for (int m = 0; m < M; ++m) {
    const T* qv = reinterpret_cast<const T*>(a.q) + (size_t)t * a.q_stride + (size_t)(h * M + m) * Dk;
    const int kh = g * M + m;
    float qr[KPL], acc[VPL];
#pragma unroll
    for (int j = 0; j < KPL; ++j) {
      const int d = lane + 32 * j;
      qr[j] = d < Dk ? to_f32(qv[d]) : 0.f;
    }
#pragma unroll
    for (int j = 0; j < VPL; ++j) acc[j] = 0.f;
    float mx = -INFINITY, l = 0.f;
    for (int s = lo; s <= pos; ++s) {
      const int page = bt[s / a.page_size], in_page = s % a.page_size;
      const T* kv = kp + (((size_t)page * (a.G * M) + kh) * a.page_size + in_page) * Dk;
      const T* vv = vp + (((size_t)page * a.G + g) * a.page_size + in_page) * Dv;
      float part = 0.f;
#pragma unroll
      for (int j = 0; j < KPL; ++j) {
        const int d = lane + 32 * j;
        if (d < Dk) part += qr[j] * to_f32(kv[d]);
      }
      const float score = warp_sum(part) * a.scale;
      const float m_new = fmaxf(mx, score);
      const float corr = expf(mx - m_new);   // exp(-inf) = 0 on the first key
      const float p = expf(score - m_new);
      l = l * corr + p;
#pragma unroll
      for (int j = 0; j < VPL; ++j) {
        const int d = lane + 32 * j;
        if (d < Dv) acc[j] = acc[j] * corr + p * to_f32(vv[d]);
      }
      mx = m_new;
    }
    if (a.sink != nullptr) {
      // the sink has no key and no value: it only joins the denominator
      const float sk = a.sink[h];
      const float m_new = fmaxf(mx, sk);
      const float corr = expf(mx - m_new);
      l = l * corr + expf(sk - m_new);
#pragma unroll
      for (int j = 0; j < VPL; ++j) acc[j] *= corr;
    }
    const float wgt = (m == 0 ? 1.0f : a.coef) / l;
#pragma unroll
    for (int j = 0; j < VPL; ++j) total[j] += acc[j] * wgt;
  }
  float mul = a.out_scale;
  if (a.unit_norm) {
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < VPL; ++j) ss += total[j] * total[j];   // lanes past Dv hold zeros
    ss = warp_sum(ss);
    mul *= 1.0f / sqrtf(ss / (float)Dv + a.eps);
  }
#pragma unroll
  for (int j = 0; j < VPL; ++j) {
    const int d = lane + 32 * j;
    if (d < Dv) o[d] = from_f32<T>(total[j] * mul);
  }
}

// a [T, H, M, Dv] float: the maps' outputs; out [T, H, Dv] = (a_0 + coef * sum_{m>0} a_m), optionally divided by
// its root mean square, times out_scale.  One warp per (token, head).
template <typename T>
__global__ void __launch_bounds__(128)
maps_combine_kernel(const float* __restrict__ a, T* __restrict__ out, const int* __restrict__ tok_seq, int n_tokens, int H,
                    int M, int Dv, float coef, int unit_norm, float eps, float out_scale) {
  pdl_wait();
  pdl_trigger();
  const int lane = threadIdx.x & 31;
  const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (w >= (long long)n_tokens * H) return;
  const int t = (int)(w / H);
  T* o = out + (size_t)w * Dv;
  if (tok_seq[t] < 0) {
    for (int d = lane; d < Dv; d += 32) o[d] = from_f32<T>(0.f);
    return;
  }
  const float* src = a + (size_t)w * M * Dv;
  float total[AM_MAX_DIM / 32];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < AM_MAX_DIM / 32; ++j) {
    const int d = lane + 32 * j;
    float v = 0.f;
    if (d < Dv) {
      v = src[d];
      for (int m = 1; m < M; ++m) v += coef * src[(size_t)m * Dv + d];
    }
    total[j] = v;
    ss += v * v;
  }
  float mul = out_scale;
  if (unit_norm) mul *= 1.0f / sqrtf(warp_sum(ss) / (float)Dv + eps);
#pragma unroll
  for (int j = 0; j < AM_MAX_DIM / 32; ++j) {
    const int d = lane + 32 * j;
    if (d < Dv) o[d] = from_f32<T>(total[j] * mul);
  }
}

AB_API int ab_maps_combine(const float* a, void* out, int dtype, const int* tok_seq, int n_tokens, int H, int M, int Dv,
                           float coef, int unit_norm, float eps, float out_scale, cudaStream_t stream) {
  if (n_tokens <= 0) return AB_OK;
  if (H <= 0 || M <= 0 || Dv <= 0 || Dv > AM_MAX_DIM) return AB_BAD_ARG;
  const long long warps = (long long)n_tokens * H;
  const unsigned blocks = (unsigned)((warps + 3) / 4);
  if (dtype == AB_F32)
    ab_launch(maps_combine_kernel<float>, dim3(blocks), dim3(128), 0, stream, a, (float*)out, tok_seq, n_tokens, H, M, Dv,
              coef, unit_norm, eps, out_scale);
  else if (dtype == AB_BF16)
    ab_launch(maps_combine_kernel<bf16>, dim3(blocks), dim3(128), 0, stream, a, (bf16*)out, tok_seq, n_tokens, H, M, Dv,
              coef, unit_norm, eps, out_scale);
  else
    return AB_BAD_ARG;
  return ab_launch_status();
}

AB_API int ab_attention_prepare_opts(void* buf, int dtype, int stride, int off_q, int off_k, int off_v, int n_q, int n_k,
                                     int n_v, int Dk, int Dv, const float* q_weight, const float* k_weight, float eps,
                                     const float* cos_t, const float* sin_t, int n_rot, int pairing, const int* tok_pos,
                                     const int* tok_seq, const int* block_table, int table_width, void* k_pages,
                                     void* v_pages, int page_size, int n_tokens, int write_cache, const float* bias,
                                     int v_norm, int v_side_by_side, cudaStream_t stream);

AB_API int ab_attention_prepare(void* buf, int dtype, int stride, int off_q, int off_k, int off_v, int n_q, int n_k,
                                int n_v, int Dk, int Dv, const float* q_weight, const float* k_weight, float eps,
                                const float* cos_t, const float* sin_t, int n_rot, int pairing, const int* tok_pos,
                                const int* tok_seq, const int* block_table, int table_width, void* k_pages,
                                void* v_pages, int page_size, int n_tokens, int write_cache, const float* bias,
                                cudaStream_t stream) {
  return ab_attention_prepare_opts(buf, dtype, stride, off_q, off_k, off_v, n_q, n_k, n_v, Dk, Dv, q_weight, k_weight, eps,
                                   cos_t, sin_t, n_rot, pairing, tok_pos, tok_seq, block_table, table_width, k_pages,
                                   v_pages, page_size, n_tokens, write_cache, bias, 0, 0, stream);
}

// `v_norm`: value vectors are divided by their root mean square before they are stored; `v_side_by_side`: value pages
// [n_pages, 1, page, n_v * Dv].
AB_API int ab_attention_prepare_opts(void* buf, int dtype, int stride, int off_q, int off_k, int off_v, int n_q, int n_k,
                                     int n_v, int Dk, int Dv, const float* q_weight, const float* k_weight, float eps,
                                     const float* cos_t, const float* sin_t, int n_rot, int pairing, const int* tok_pos,
                                     const int* tok_seq, const int* block_table, int table_width, void* k_pages,
                                     void* v_pages, int page_size, int n_tokens, int write_cache, const float* bias,
                                     int v_norm, int v_side_by_side, cudaStream_t stream) {
  if (n_tokens <= 0) return AB_OK;
  if (Dk <= 0 || Dk > AM_MAX_DIM || Dv <= 0 || n_q < 0 || n_k < 0 || n_v < 0 || page_size <= 0) return AB_BAD_ARG;
  if (n_rot < 0 || n_rot > Dk || (n_rot & 1) || pairing < 0 || pairing > 1) return AB_BAD_ARG;
  if (!cos_t || !sin_t || n_rot == 0) { cos_t = sin_t = nullptr; n_rot = 0; }
  PrepareArgs a{buf, stride, off_q, off_k, off_v, n_q, n_k, n_v, Dk, Dv, q_weight, k_weight, eps, cos_t, sin_t, n_rot,
                pairing, tok_pos, tok_seq, block_table, table_width, k_pages, v_pages, page_size, n_tokens, write_cache,
                bias, v_norm ? 1 : 0, v_side_by_side ? 1 : 0};
  const long long warps = (long long)n_tokens * (n_q + n_k + n_v);
  const unsigned blocks = (unsigned)((warps + 3) / 4);
  const bool pieces = !v_norm && dtype == AB_BF16 && Dk % 8 == 0 && Dv % 8 == 0 && stride % 8 == 0 && off_q % 8 == 0 &&
                      off_k % 8 == 0 && off_v % 8 == 0 && (n_rot == 0 || pairing == 0 || n_rot % 16 == 0);
  if (pieces) {
    const int P = Dk / 8, vpw = 32 / P;
    const long long qk_warps = ((long long)n_tokens * (n_q + n_k) + vpw - 1) / vpw;
    const long long v_warps = ((long long)n_tokens * n_v * (Dv / 8) + 31) / 32;
    ab_launch(attention_prepare_vec_kernel, dim3((unsigned)((qk_warps + v_warps + 3) / 4)), dim3(128), 0, stream, a, P, vpw,
              qk_warps);
    return ab_launch_status();
  }
  if (dtype == AB_F32) ab_launch(attention_prepare_kernel<float>, dim3(blocks), dim3(128), 0, stream, a);
  else if (dtype == AB_BF16) ab_launch(attention_prepare_kernel<bf16>, dim3(blocks), dim3(128), 0, stream, a);
  else return AB_BAD_ARG;
  return ab_launch_status();
}

template <typename T>
static int launch_attend(const AttendArgs& a, cudaStream_t stream) {
  const long long warps = (long long)a.n_tokens * a.H;
  const unsigned blocks = (unsigned)((warps + 3) / 4);
  const int kc = a.Dk <= 64 ? 2 : (a.Dk <= 128 ? 4 : 8), vc = a.Dv <= 64 ? 2 : (a.Dv <= 128 ? 4 : 8);
#define AB_GO(KPL, VPL) ab_launch(attention_maps_kernel<T, KPL, VPL>, dim3(blocks), dim3(128), 0, stream, a)
  if (kc == 2 && vc == 2) AB_GO(2, 2);
  else if (kc == 2 && vc == 4) AB_GO(2, 4);
  else if (kc == 2) AB_GO(2, 8);
  else if (kc == 4 && vc == 2) AB_GO(4, 2);
  else if (kc == 4 && vc == 4) AB_GO(4, 4);
  else if (kc == 4) AB_GO(4, 8);
  else if (vc == 2) AB_GO(8, 2);
  else if (vc == 4) AB_GO(8, 4);
  else AB_GO(8, 8);
#undef AB_GO
  return ab_launch_status();
}

AB_API int ab_attention_maps(const void* q, int q_stride, void* out, int dtype, const void* k_pages,
                             const void* v_pages, const int* block_table, int table_width, const int* tok_pos,
                             const int* tok_seq, int n_tokens, int H, int G, int M, int Dk, int Dv, int page_size,
                             float scale, int window, const float* sink, float coef, int unit_norm, float eps,
                             float out_scale, cudaStream_t stream) {
  if (n_tokens <= 0) return AB_OK;
  if (Dk <= 0 || Dk > AM_MAX_DIM || Dv <= 0 || Dv > AM_MAX_DIM || H <= 0 || G <= 0 || H % G || M <= 0 || page_size <= 0)
    return AB_BAD_ARG;
  AttendArgs a{q, q_stride, out, k_pages, v_pages, block_table, table_width, tok_pos, tok_seq, n_tokens, H, G, M, Dk,
               Dv, page_size, scale, window, sink, coef, unit_norm, eps, out_scale};
  if (dtype == AB_F32) return launch_attend<float>(a, stream);
  if (dtype == AB_BF16) return launch_attend<bf16>(a, stream);
  return AB_BAD_ARG;
}


// ---------------------------------------------------------------------------
// softmax weights mixed across heads
// ---------------------------------------------------------------------------
struct TalkArgs {
  const void* q; int q_stride;      // query vector x of token t at q + t*q_stride + x*Dk; it reads key head x % G
  float* A;                         // [T, H, G*Dv]
  const void* k_pages;              // [n_pages, G, page, Dk]
  const void* v_pages;              // [n_pages, 1, page, G*Dv]
  const int* block_table; int table_width;
  const int* tok_pos; const int* tok_seq;
  int n_tokens, H, G, Dk, Dv, page_size;
  float scale; int window;
};

template <typename T, int KPL, int VPL>
__global__ void __launch_bounds__(128)
talk_attend_kernel(TalkArgs a) {
  pdl_wait();
  pdl_trigger();
  const int lane = threadIdx.x & 31;
  const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (w >= (long long)a.n_tokens * a.H) return;
  const int t = (int)(w / a.H), x = (int)(w - (long long)t * a.H);
  const int Dk = a.Dk, W = a.G * a.Dv;
  float* o = a.A + (size_t)w * W;
  const int b = a.tok_seq[t];
  if (b < 0) {
    for (int d = lane; d < W; d += 32) o[d] = 0.f;
    return;
  }
  const int pos = a.tok_pos[t];
  const int kh = x % a.G;
  const int lo = (a.window > 0 && pos - a.window + 1 > 0) ? pos - a.window + 1 : 0;
  const int* bt = a.block_table + (size_t)b * a.table_width;
  const T* kp = reinterpret_cast<const T*>(a.k_pages);
  const T* vp = reinterpret_cast<const T*>(a.v_pages);
  const T* qv = reinterpret_cast<const T*>(a.q) + (size_t)t * a.q_stride + (size_t)x * Dk;
  float qr[KPL], acc[VPL];
#pragma unroll
  for (int j = 0; j < KPL; ++j) {
    const int d = lane + 32 * j;
    qr[j] = d < Dk ? to_f32(qv[d]) : 0.f;
  }
#pragma unroll
  for (int j = 0; j < VPL; ++j) acc[j] = 0.f;
  float mx = -INFINITY, l = 0.f;
  for (int s = lo; s <= pos; ++s) {
    const int page = bt[s / a.page_size], in_page = s % a.page_size;
    const T* kv = kp + (((size_t)page * a.G + kh) * a.page_size + in_page) * Dk;
    const T* vv = vp + ((size_t)page * a.page_size + in_page) * W;
    float part = 0.f;
#pragma unroll
    for (int j = 0; j < KPL; ++j) {
      const int d = lane + 32 * j;
      if (d < Dk) part += qr[j] * to_f32(kv[d]);
    }
    const float score = warp_sum(part) * a.scale;
    const float m_new = fmaxf(mx, score);
    const float corr = expf(mx - m_new);   // exp(-inf) = 0 on the first key
    const float p = expf(score - m_new);
    l = l * corr + p;
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      const int d = lane + 32 * j;
      if (d < W) acc[j] = acc[j] * corr + p * to_f32(vv[d]);
    }
    mx = m_new;
  }
  const float inv = 1.0f / l;
#pragma unroll
  for (int j = 0; j < VPL; ++j) {
    const int d = lane + 32 * j;
    if (d < W) o[d] = acc[j] * inv;
  }
}

// out[t, h, d] = gate * sum_g T[h, g] A[t, x(g), c(h)*Dv + d], x(g) = (g % R) * G + g / R, c(h) = h / R, R = H / G;
// gate = sigmoid(gate_rows[t*gate_stride + h*Dv + d]) or 1.  A thread per VEC neighbouring columns c*Dv + d of a
// token's rows of A (VEC = 4 where Dv is a multiple of 4): it reads those columns of all H rows once (neighbouring
// threads neighbouring addresses) and writes the R heads of group c, four at a time.  The mixing matrix and the
// head that row x belongs to wait in shared memory (`talk_smem`: the matrix fits).
template <typename T, int VEC>
__global__ void __launch_bounds__(128)
talk_combine_kernel(const float* __restrict__ A, const float* __restrict__ talk, const T* __restrict__ gate_rows,
                    int gate_stride, T* __restrict__ out, const int* __restrict__ tok_seq, int n_tokens, int H, int G,
                    int Dv, int talk_smem) {
  extern __shared__ float tc_smem[];       // head of row x [H] (as int), then talk [H*H] (if talk_smem)
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  const int W = G * Dv, R = H / G;
  const int col = (blockIdx.y * blockDim.x + threadIdx.x) * VEC;
  const bool live = tok_seq[t] >= 0;
  int* head_of = reinterpret_cast<int*>(tc_smem);
  float* tks = tc_smem + H;
  if (live) {
    for (int x = threadIdx.x; x < H; x += blockDim.x) head_of[x] = (x % G) * R + x / G;
    if (talk_smem)
      for (int i = threadIdx.x; i < H * H; i += blockDim.x) tks[i] = talk[i];
  }
  __syncthreads();
  if (col >= W) return;
  const int c = col / Dv, d = col - c * Dv;
  if (!live) {
    for (int j = 0; j < R; ++j)
      for (int v = 0; v < VEC; ++v) out[((size_t)t * H + c * R + j) * Dv + d + v] = from_f32<T>(0.f);
    return;
  }
  const float* tk = talk_smem ? tks : talk;
  const float* At = A + (size_t)t * H * W + col;
  for (int j0 = 0; j0 < R; j0 += 4) {
    float acc[4][VEC];
#pragma unroll
    for (int jj = 0; jj < 4; ++jj)
#pragma unroll
      for (int v = 0; v < VEC; ++v) acc[jj][v] = 0.f;
#pragma unroll 4
    for (int x = 0; x < H; ++x) {
      float a[VEC];
      if (VEC == 4) {
        const float4 raw = *reinterpret_cast<const float4*>(At + (size_t)x * W);
        a[0] = raw.x; a[VEC > 1 ? 1 : 0] = raw.y; a[VEC > 2 ? 2 : 0] = raw.z; a[VEC > 3 ? 3 : 0] = raw.w;
      } else {
        a[0] = At[(size_t)x * W];
      }
      const int g = head_of[x];
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        const float w = j0 + jj < R ? tk[(size_t)(c * R + j0 + jj) * H + g] : 0.f;
#pragma unroll
        for (int v = 0; v < VEC; ++v) acc[jj][v] = fmaf(w, a[v], acc[jj][v]);
      }
    }
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) {
      if (j0 + jj >= R) break;
      const int h = c * R + j0 + jj;
#pragma unroll
      for (int v = 0; v < VEC; ++v) {
        float sum = acc[jj][v];
        if (gate_rows != nullptr)
          sum *= 1.0f / (1.0f + expf(-to_f32(gate_rows[(size_t)t * gate_stride + h * Dv + d + v])));
        out[((size_t)t * H + h) * Dv + d + v] = from_f32<T>(sum);
      }
    }
  }
}

// Merges the parts that `talk_decode` leaves: A[t, x, :] = sum_p w_p Ap[t, p, x, :] with w_p = exp2(m_p - m) / sum_p
// l_p exp2(m_p - m), m the largest m_p (a part without keys has l = 0 and is left out).  A block per (token, x).
__global__ void __launch_bounds__(128)
talk_merge_kernel(const float* __restrict__ Ap, const float* __restrict__ ml, float* __restrict__ A, int parts, int H,
                  int W) {
  __shared__ float wts[64];
  pdl_wait();
  pdl_trigger();
  const int x = blockIdx.x % H, t = blockIdx.x / H;
  const float* mlx = ml + ((size_t)t * parts * H + x) * 2;
  if (threadIdx.x < 32) {
    float m = -INFINITY;
    for (int p = threadIdx.x; p < parts; p += 32)
      if (mlx[(size_t)p * H * 2 + 1] > 0.f) m = fmaxf(m, mlx[(size_t)p * H * 2]);
    m = warp_max(m);
    float l = 0.f;
    for (int p = threadIdx.x; p < parts; p += 32) {
      const float lp = mlx[(size_t)p * H * 2 + 1];
      if (lp > 0.f) l += lp * exp2f(mlx[(size_t)p * H * 2] - m);
    }
    l = warp_sum(l);
    for (int p = threadIdx.x; p < parts; p += 32) {
      const float lp = mlx[(size_t)p * H * 2 + 1];
      wts[p] = (lp > 0.f && l > 0.f) ? exp2f(mlx[(size_t)p * H * 2] - m) / l : 0.f;
    }
  }
  __syncthreads();
  const float* src = Ap + ((size_t)t * parts * H + x) * W;
  float* dst = A + ((size_t)t * H + x) * W;
  for (int col = threadIdx.x * 4; col < W; col += blockDim.x * 4) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int p = 0; p < parts; ++p) {
      const float w = wts[p];
      if (w != 0.f) {
        const float4 v = *reinterpret_cast<const float4*>(src + (size_t)p * H * W + col);
        acc.x = fmaf(w, v.x, acc.x); acc.y = fmaf(w, v.y, acc.y); acc.z = fmaf(w, v.z, acc.z); acc.w = fmaf(w, v.w, acc.w);
      }
    }
    *reinterpret_cast<float4*>(dst + col) = acc;
  }
}

// One token per sequence: the keys of a token are cut into `parts` runs of `pages_per_part` pages, and a CTA takes
// (token, key head kh, part, up to 4 of the R query vectors that read kh, up to 512 of the G*Dv value columns), so that
// a step of few tokens fills the device.  It leaves sums of exp2(score - m) * v in Ap [T, parts, H, W] and (m, l) in
// ml [T, parts, H, 2]; `talk_combine` merges the parts.  Scores are float32 sums over the key's dims in order; a
// thread owns 4 neighbouring value columns.  The geometry depends on the block table's width alone, the lengths are
// read from device memory: a captured step stays valid while its sequences grow.
#define TD_KEYS 64
#define TD_RC 4
#define TD_COLS 512
template <typename T>
__global__ void __launch_bounds__(128)
talk_decode_kernel(TalkArgs a, float* __restrict__ ml, int parts, int pages_per_part, int r_chunks, int col_blocks) {
  extern __shared__ __align__(16) unsigned char td_raw[];
  pdl_wait();
  pdl_trigger();
  const int Dk = a.Dk, W = a.G * a.Dv, R = a.H / a.G, H = a.H;
  float* qs = reinterpret_cast<float*>(td_raw);             // [TD_RC][Dk]
  float* ps = qs + TD_RC * Dk;                               // [TD_RC][TD_KEYS]
  float* corr = ps + TD_RC * TD_KEYS;                        // [TD_RC]
  T* ks = reinterpret_cast<T*>(corr + TD_RC);                // [TD_KEYS][Dk + pad]
  const int kpitch = Dk + (16 / (int)sizeof(T));
  int idx = blockIdx.x;
  const int cb = idx % col_blocks; idx /= col_blocks;
  const int rc = idx % r_chunks; idx /= r_chunks;
  const int p = idx % parts; idx /= parts;
  const int kh = idx % a.G;
  const int t = idx / a.G;
  const int b = a.tok_seq[t];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int j0 = rc * TD_RC, nr = min(TD_RC, R - j0);       // query vectors x = (j0 + r) * G + kh, r < nr
  const int col = cb * TD_COLS + tid * 4;
  float* mlo = ml + ((size_t)t * parts + p) * H * 2;
  if (b < 0) {
    if (cb == 0 && tid < nr) { mlo[((j0 + tid) * a.G + kh) * 2] = -INFINITY; mlo[((j0 + tid) * a.G + kh) * 2 + 1] = 0.f; }
    return;
  }
  const int pos = a.tok_pos[t];
  const int lo = (a.window > 0 && pos - a.window + 1 > 0) ? pos - a.window + 1 : 0;
  const int page0 = lo / a.page_size + p * pages_per_part;
  const int page1 = min(page0 + pages_per_part, pos / a.page_size + 1);
  if (page0 >= page1) {
    if (cb == 0 && tid < nr) { mlo[((j0 + tid) * a.G + kh) * 2] = -INFINITY; mlo[((j0 + tid) * a.G + kh) * 2 + 1] = 0.f; }
    return;
  }
  const T* qrow = reinterpret_cast<const T*>(a.q) + (size_t)t * a.q_stride;
  for (int i = tid; i < nr * Dk; i += 128) {
    const int r = i / Dk, d = i - r * Dk;
    qs[i] = to_f32(qrow[(size_t)((j0 + r) * a.G + kh) * Dk + d]) * a.scale * 1.4426950408889634f;
  }
  const int* bt = a.block_table + (size_t)b * a.table_width;
  const T* kp = reinterpret_cast<const T*>(a.k_pages);
  const T* vp = reinterpret_cast<const T*>(a.v_pages);
  float acc[TD_RC][4];
#pragma unroll
  for (int r = 0; r < TD_RC; ++r) acc[r][0] = acc[r][1] = acc[r][2] = acc[r][3] = 0.f;
  float m_run = -INFINITY, l_run = 0.f;      // of row r = warp (a warp per query vector), kept by every lane
  const bool own_col = col < W && col < (cb + 1) * TD_COLS;
  for (int pg = page0; pg < page1; ++pg) {
    const int page = bt[pg];
    const int key0 = pg * a.page_size;
    const int n_keys = min(a.page_size, pos - key0 + 1);
    {
      // ask the L2 for what comes after the scores: this page's value rows (the CTA's columns), and the next
      // page's keys, 128 bytes per request
      const int first = cb * TD_COLS, n_col = min(TD_COLS, W - first);
      const int lines = (n_col * (int)sizeof(T) + 127) / 128;
      const char* vbase = reinterpret_cast<const char*>(vp + ((size_t)page * a.page_size) * W + first);
      for (int i = tid; i < n_keys * lines; i += 128) {
        const int k = i / lines, ln = i - k * lines;
        asm volatile("prefetch.global.L2 [%0];" ::"l"(vbase + (size_t)k * W * sizeof(T) + (size_t)ln * 128));
      }
      if (pg + 1 < page1) {
        const char* kbase = reinterpret_cast<const char*>(kp + ((size_t)bt[pg + 1] * a.G + kh) * a.page_size * Dk);
        const int kbytes = min(a.page_size, pos - key0 - a.page_size + 1) * Dk * (int)sizeof(T);
        for (int i = tid * 128; i < kbytes; i += 128 * 128) asm volatile("prefetch.global.L2 [%0];" ::"l"(kbase + i));
      }
    }
    __syncthreads();                          // the tile and the weights of the page before are done with
    {
      // the page's keys of head kh, 16 bytes at a time
      const T* src = kp + ((size_t)page * a.G + kh) * a.page_size * Dk;
      constexpr int PER = 16 / (int)sizeof(T);
      const int cpr = Dk / PER;
      for (int c = tid; c < n_keys * cpr; c += 128) {
        const int k = c / cpr, cc = c - k * cpr;
        *reinterpret_cast<uint4*>(ks + k * kpitch + cc * PER) = *reinterpret_cast<const uint4*>(src + (size_t)k * Dk + cc * PER);
      }
    }
    __syncthreads();
    // scores: thread (key, half) takes the rows r = half and half + 2, the key's numbers 16 bytes at a time
    {
      const int k = tid & 63, half = tid >> 6;
      constexpr int PER = 16 / (int)sizeof(T);
      float s0 = 0.f, s1 = 0.f;
      const bool seen = k < n_keys && key0 + k >= lo;
      if (seen && half < nr) {
        const T* kr = ks + k * kpitch;
        const float* q0 = qs + half * Dk;
        const float* q1 = qs + (half + 2 < nr ? half + 2 : half) * Dk;
        for (int d = 0; d < Dk; d += PER) {
          const uint4 raw = *reinterpret_cast<const uint4*>(kr + d);
          float kv[PER];
          if (sizeof(T) == 2) {
            kv[0] = __uint_as_float(raw.x << 16); kv[1] = __uint_as_float(raw.x & 0xffff0000u);
            kv[2] = __uint_as_float(raw.y << 16); kv[3] = __uint_as_float(raw.y & 0xffff0000u);
            if (PER > 4) {
              kv[PER - 4] = __uint_as_float(raw.z << 16); kv[PER - 3] = __uint_as_float(raw.z & 0xffff0000u);
              kv[PER - 2] = __uint_as_float(raw.w << 16); kv[PER - 1] = __uint_as_float(raw.w & 0xffff0000u);
            }
          } else {
            kv[0] = __uint_as_float(raw.x); kv[1] = __uint_as_float(raw.y);
            kv[2] = __uint_as_float(raw.z); kv[3] = __uint_as_float(raw.w);
          }
#pragma unroll
          for (int i = 0; i < PER; ++i) {
            s0 = fmaf(q0[d + i], kv[i], s0);
            s1 = fmaf(q1[d + i], kv[i], s1);
          }
        }
      }
      if (half < nr) ps[half * TD_KEYS + k] = seen ? s0 : -INFINITY;
      if (half + 2 < nr) ps[(half + 2) * TD_KEYS + k] = seen ? s1 : -INFINITY;
    }
    __syncthreads();
    // a warp per row: the running maximum and sum, the weights in place of the scores
    if (warp < nr) {
      const float s0 = ps[warp * TD_KEYS + lane], s1 = ps[warp * TD_KEYS + lane + 32];
      const float m_new = fmaxf(m_run, warp_max(fmaxf(s0, s1)));
      const float c0 = (m_new == -INFINITY) ? 1.f : exp2f(m_run - m_new);
      const float p0 = (s0 == -INFINITY) ? 0.f : exp2f(s0 - m_new), p1 = (s1 == -INFINITY) ? 0.f : exp2f(s1 - m_new);
      ps[warp * TD_KEYS + lane] = p0;
      ps[warp * TD_KEYS + lane + 32] = p1;
      l_run = l_run * c0 + warp_sum(p0 + p1);
      m_run = m_new;
      if (lane == 0) corr[warp] = c0;
    }
    __syncthreads();
    if (own_col) {
#pragma unroll
      for (int r = 0; r < TD_RC; ++r) {
        const float c0 = r < nr ? corr[r] : 1.f;
        acc[r][0] *= c0; acc[r][1] *= c0; acc[r][2] *= c0; acc[r][3] *= c0;
      }
      const T* vrow = vp + ((size_t)page * a.page_size) * W + col;
      // the values of 16 keys are asked for at once (keys past the page's last have weight 0)
      for (int k0 = 0; k0 < n_keys; k0 += 16) {
        float4 vals[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          vals[i] = make_float4(0.f, 0.f, 0.f, 0.f);
          if (k0 + i < n_keys) {
            if (sizeof(T) == 2) {
              const uint2 raw = *reinterpret_cast<const uint2*>(vrow + (size_t)(k0 + i) * W);
              vals[i] = make_float4(__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xffff0000u),
                                    __uint_as_float(raw.y << 16), __uint_as_float(raw.y & 0xffff0000u));
            } else {
              vals[i] = *reinterpret_cast<const float4*>(vrow + (size_t)(k0 + i) * W);
            }
          }
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) {
#pragma unroll
          for (int r = 0; r < TD_RC; ++r) {
            const float pk = ps[r * TD_KEYS + k0 + i];      // rows past nr hold what was there: their sums are not stored
            acc[r][0] = fmaf(pk, vals[i].x, acc[r][0]);
            acc[r][1] = fmaf(pk, vals[i].y, acc[r][1]);
            acc[r][2] = fmaf(pk, vals[i].z, acc[r][2]);
            acc[r][3] = fmaf(pk, vals[i].w, acc[r][3]);
          }
        }
      }
    }
  }
  if (cb == 0 && warp < nr && lane == 0) {
    mlo[((j0 + warp) * a.G + kh) * 2] = m_run;
    mlo[((j0 + warp) * a.G + kh) * 2 + 1] = l_run;
  }
  if (own_col) {
#pragma unroll
    for (int r = 0; r < TD_RC; ++r)
      if (r < nr) {
        float* o = a.A + (((size_t)t * parts + p) * H + (j0 + r) * a.G + kh) * W + col;
        *reinterpret_cast<float4*>(o) = make_float4(acc[r][0], acc[r][1], acc[r][2], acc[r][3]);
      }
  }
}

template <typename T>
static int launch_talk(const TalkArgs& a, cudaStream_t stream) {
  const long long warps = (long long)a.n_tokens * a.H;
  const unsigned blocks = (unsigned)((warps + 3) / 4);
  const int W = a.G * a.Dv;
  const int kc = a.Dk <= 64 ? 2 : (a.Dk <= 128 ? 4 : 8);
#define AB_GO(KPL, VPL) ab_launch(talk_attend_kernel<T, KPL, VPL>, dim3(blocks), dim3(128), 0, stream, a)
#define AB_V(KPL)                                   \
  if (W <= 64) AB_GO(KPL, 2);                       \
  else if (W <= 128) AB_GO(KPL, 4);                 \
  else if (W <= 256) AB_GO(KPL, 8);                 \
  else if (W <= 512) AB_GO(KPL, 16);                \
  else if (W <= 1024) AB_GO(KPL, 32);               \
  else AB_GO(KPL, 64);
  if (kc == 2) { AB_V(2) } else if (kc == 4) { AB_V(4) } else { AB_V(8) }
#undef AB_V
#undef AB_GO
  return ab_launch_status();
}

#define TALK_MAX_ROW 2048      // G * Dv: the numbers of a token's values that a warp holds sums for

AB_API int ab_talk_max_row() { return TALK_MAX_ROW; }

AB_API int ab_talk_attend(const void* q, int q_stride, float* A, int dtype, const void* k_pages, const void* v_pages,
                          const int* block_table, int table_width, const int* tok_pos, const int* tok_seq, int n_tokens,
                          int H, int G, int Dk, int Dv, int page_size, float scale, int window, cudaStream_t stream) {
  if (n_tokens <= 0) return AB_OK;
  if (Dk <= 0 || Dk > AM_MAX_DIM || Dv <= 0 || H <= 0 || G <= 0 || H % G || (long long)G * Dv > TALK_MAX_ROW ||
      page_size <= 0)
    return AB_BAD_ARG;
  TalkArgs a{q, q_stride, A, k_pages, v_pages, block_table, table_width, tok_pos, tok_seq, n_tokens, H, G, Dk, Dv,
             page_size, scale, window};
  if (dtype == AB_F32) return launch_talk<float>(a, stream);
  if (dtype == AB_BF16) return launch_talk<bf16>(a, stream);
  return AB_BAD_ARG;
}

AB_API int ab_talk_combine(const float* A, const float* talk, const void* gate_rows, int gate_stride, void* out, int dtype,
                           const int* tok_seq, int n_tokens, int H, int G, int Dv, cudaStream_t stream) {
  if (n_tokens <= 0) return AB_OK;
  if (H <= 0 || G <= 0 || H % G || Dv <= 0 || !tok_seq) return AB_BAD_ARG;
  const int W = G * Dv;
  size_t smem = (size_t)H * sizeof(float);
  const int talk_smem = (size_t)H * H * sizeof(float) + smem <= 40 * 1024 ? 1 : 0;
  if (talk_smem) smem += (size_t)H * H * sizeof(float);
  if (smem > 48 * 1024) return AB_BAD_ARG;
  const int vec = (Dv % 4 == 0) ? 4 : 1;
  dim3 grid((unsigned)n_tokens, (unsigned)((W / vec + 127) / 128));
#define AB_GO(T, VEC)                                                                                             \
  ab_launch(talk_combine_kernel<T, VEC>, grid, dim3(128), smem, stream, A, talk, (const T*)gate_rows, gate_stride, \
            (T*)out, tok_seq, n_tokens, H, G, Dv, talk_smem)
  if (dtype == AB_F32) { if (vec == 4) AB_GO(float, 4); else AB_GO(float, 1); }
  else if (dtype == AB_BF16) { if (vec == 4) AB_GO(bf16, 4); else AB_GO(bf16, 1); }
  else return AB_BAD_ARG;
#undef AB_GO
  return ab_launch_status();
}

// A[t, x, :] from the `parts` partial rows Ap [T, parts, H, W] and their (m, l) in ml [T, parts, H, 2]; W a multiple
// of 4, up to 64 parts.
AB_API int ab_talk_merge(const float* Ap, const float* ml, float* A, int parts, int n_tokens, int H, int W,
                         cudaStream_t stream) {
  if (n_tokens <= 0) return AB_OK;
  if (parts < 1 || parts > 64 || H <= 0 || W <= 0 || W % 4 || (long long)n_tokens * H > 0x7fffffffLL) return AB_BAD_ARG;
  ab_launch(talk_merge_kernel, dim3((unsigned)(n_tokens * H)), dim3(128), 0, stream, Ap, ml, A, parts, H, W);
  return ab_launch_status();
}

// The decode form: one token per sequence, the keys in `parts` runs of `pages_per_part` pages (see the kernel).
// Ap float [T, parts, H, G*Dv], ml float [T, parts, H, 2].  Sizes: Dk in 16-byte pieces, G*Dv a multiple of 4.
AB_API int ab_talk_decode(const void* q, int q_stride, float* Ap, float* ml, int parts, int pages_per_part, int dtype,
                          const void* k_pages, const void* v_pages, const int* block_table, int table_width,
                          const int* tok_pos, const int* tok_seq, int n_tokens, int H, int G, int Dk, int Dv,
                          int page_size, float scale, int window, cudaStream_t stream) {
  if (n_tokens <= 0) return AB_OK;
  if (Dk <= 0 || Dv <= 0 || H <= 0 || G <= 0 || H % G || page_size != TD_KEYS || parts < 1 || pages_per_part < 1)
    return AB_BAD_ARG;
  const int W = G * Dv, R = H / G;
  const int per = dtype == AB_BF16 ? 8 : 4;
  if (Dk % per || W % 4) return AB_BAD_ARG;
  const int r_chunks = (R + TD_RC - 1) / TD_RC, col_blocks = (W + TD_COLS - 1) / TD_COLS;
  const long long blocks = (long long)n_tokens * G * parts * r_chunks * col_blocks;
  if (blocks > 0x7fffffffLL) return AB_BAD_ARG;
  TalkArgs a{q, q_stride, Ap, k_pages, v_pages, block_table, table_width, tok_pos, tok_seq, n_tokens, H, G, Dk, Dv,
             page_size, scale, window};
  const size_t esz = dtype == AB_BF16 ? 2 : 4;
  const size_t smem = (size_t)(TD_RC * Dk + TD_RC * TD_KEYS + TD_RC) * sizeof(float) + (size_t)TD_KEYS * (Dk + 16 / esz) * esz;
#define AB_GO(T)                                                                                                    \
  {                                                                                                                 \
    if (smem > 48 * 1024) {                                                                                         \
      cudaError_t e = cudaFuncSetAttribute(talk_decode_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,      \
                                           (int)smem);                                                              \
      if (e != cudaSuccess) return AB_CUDA_ERR + (int)e;                                                            \
    }                                                                                                               \
    ab_launch(talk_decode_kernel<T>, dim3((unsigned)blocks), dim3(128), smem, stream, a, ml, parts, pages_per_part,  \
              r_chunks, col_blocks);                                                                                \
  }
  if (dtype == AB_BF16) AB_GO(bf16)
  else if (dtype == AB_F32) AB_GO(float)
  else return AB_BAD_ARG;
#undef AB_GO
  return ab_launch_status();
}
