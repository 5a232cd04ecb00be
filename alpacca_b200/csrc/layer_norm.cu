// Layer norm with weight and bias on the float32 residual stream:
//
//   LN(v)[j] = (v[j] - mean(v)) / sqrt(mean((v - mean(v))^2) + eps) * w[j] + b[j]
//
//   layer_norm            x += delta (if given and no rows are picked); out[i] = cast(LN(x[row_i]))
//   post_layer_norm_add   for a sub-layer whose output is normed before it joins the stream, with the next
//                         sub-layer's norm in the same kernel:
//                             y = ca * a, or y = ca * a + cb * b for two sub-layers side by side
//                             x += mult * LN_post(y);   out = cast(LN_next(x))   (if asked for)
//
// A block per row; the row waits in registers (widths that are multiples of 4 up to 8,192: every input asked for at
// once, 16 bytes per access) or in shared memory between the passes (mean, then squared deviations, then the result:
// the variance is taken about the mean, not as a difference of two sums).  Arithmetic is 32-bit; rows
// whose sequence index is negative (padding of a captured step) are left alone.
#include "common.cuh"
#include "launch.cuh"

// mean and 1 / sqrt(variance + eps) of the `width` numbers in `row` (shared memory)
__device__ __forceinline__ void row_moments(const float* row, int width, float eps, float* scratch, float& mean,
                                            float& inv) {
  float s = 0.f;
  for (int j = threadIdx.x; j < width; j += blockDim.x) s += row[j];
  mean = block_sum(s, scratch) / (float)width;
  float d2 = 0.f;
  for (int j = threadIdx.x; j < width; j += blockDim.x) {
    const float d = row[j] - mean;
    d2 += d * d;
  }
  inv = 1.0f / sqrtf(block_sum(d2, scratch) / (float)width + eps);
}

template <typename TD, typename TO>
__global__ void layer_norm_kernel(float* __restrict__ x, const TD* __restrict__ delta, const int* __restrict__ rows,
                                  const float* __restrict__ w, const float* __restrict__ b, TO* __restrict__ out,
                                  int width, float eps) {
  extern __shared__ float ln_row[];
  __shared__ float scratch[32];
  pdl_wait();
  pdl_trigger();
  const int i = blockIdx.x;
  const size_t src = (size_t)(rows != nullptr ? rows[i] : i) * width;
  for (int j = threadIdx.x; j < width; j += blockDim.x) {
    float v = x[src + j];
    if (delta != nullptr && rows == nullptr) {
      v += to_f32(delta[src + j]);
      x[src + j] = v;
    }
    ln_row[j] = v;
  }
  if (out == nullptr) return;
  __syncthreads();
  float mean, inv;
  row_moments(ln_row, width, eps, scratch, mean, inv);
  TO* o = out + (size_t)i * width;
  for (int j = threadIdx.x; j < width; j += blockDim.x) o[j] = from_f32<TO>((ln_row[j] - mean) * inv * w[j] + b[j]);
}

AB_API int ab_layer_norm(float* x, const void* delta, int delta_dtype, const int* rows, const float* w, const float* b,
                         void* out, int out_dtype, int n_rows, int width, float eps, cudaStream_t stream) {
  if (n_rows <= 0 || width <= 0) return AB_OK;
  if (!x || !w || !b) return AB_BAD_ARG;
  const size_t smem = (size_t)width * sizeof(float);
  if (smem > 200 * 1024) return AB_BAD_ARG;
  const int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
#define AB_GO(TD, TO)                                                                                              \
  {                                                                                                                \
    if (smem > 48 * 1024)                                                                                          \
      cudaFuncSetAttribute(layer_norm_kernel<TD, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);     \
    ab_launch(layer_norm_kernel<TD, TO>, dim3((unsigned)n_rows), dim3(threads), smem, stream, x, (const TD*)delta, \
              rows, w, b, (TO*)out, width, eps);                                                                   \
  }
  const bool out_f32 = out == nullptr || out_dtype == AB_F32;
  if (!out_f32 && out_dtype != AB_BF16) return AB_BAD_ARG;
  const bool d_f32 = delta == nullptr || delta_dtype == AB_F32;
  if (!d_f32 && delta_dtype != AB_BF16) return AB_BAD_ARG;
  if (d_f32) { if (out_f32) AB_GO(float, float) else AB_GO(float, bf16) }
  else { if (out_f32) AB_GO(bf16, float) else AB_GO(bf16, bf16) }
#undef AB_GO
  return ab_launch_status();
}

template <typename TA, typename TO>
__global__ void post_layer_norm_add_kernel(float* __restrict__ x, const TA* __restrict__ a, const TA* __restrict__ b,
                                           float ca, float cb, const float* __restrict__ w,
                                           const float* __restrict__ bias, float mult, const float* __restrict__ w_next,
                                           const float* __restrict__ b_next, TO* __restrict__ out,
                                           const int* __restrict__ tok_seq, int width, float eps) {
  extern __shared__ float ln_row[];
  __shared__ float scratch[32];
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  const size_t at = (size_t)t * width;
  if (tok_seq != nullptr && tok_seq[t] < 0) {
    if (out != nullptr)
      for (int j = threadIdx.x; j < width; j += blockDim.x) out[at + j] = from_f32<TO>(0.f);
    return;
  }
  for (int j = threadIdx.x; j < width; j += blockDim.x) {
    float v = ca * to_f32(a[at + j]);
    if (b != nullptr) v += cb * to_f32(b[at + j]);
    ln_row[j] = v;
  }
  __syncthreads();
  float mean, inv;
  row_moments(ln_row, width, eps, scratch, mean, inv);
  for (int j = threadIdx.x; j < width; j += blockDim.x) {     // a thread meets its own elements of the row again
    const float v = x[at + j] + mult * ((ln_row[j] - mean) * inv * w[j] + bias[j]);
    x[at + j] = v;
    ln_row[j] = v;
  }
  if (out == nullptr) return;
  __syncthreads();
  row_moments(ln_row, width, eps, scratch, mean, inv);
  for (int j = threadIdx.x; j < width; j += blockDim.x)
    out[at + j] = from_f32<TO>((ln_row[j] - mean) * inv * w_next[j] + b_next[j]);
}

// Four numbers of a row per access (widths that are multiples of 4).
template <typename T> struct LnRow4;
template <> struct LnRow4<float> {
  static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
  static __device__ __forceinline__ void store(float* p, float4 a) { *reinterpret_cast<float4*>(p) = a; }
};
template <> struct LnRow4<bf16> {
  static __device__ __forceinline__ float4 load(const bf16* p) {
    const uint2 v = *reinterpret_cast<const uint2*>(p);
    return make_float4(__uint_as_float(v.x << 16), __uint_as_float(v.x & 0xffff0000u), __uint_as_float(v.y << 16),
                       __uint_as_float(v.y & 0xffff0000u));
  }
  static __device__ __forceinline__ void store(bf16* p, float4 a) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(a.x, a.y), hi = __floats2bfloat162_rn(a.z, a.w);
    uint2 v;
    v.x = *reinterpret_cast<const unsigned*>(&lo);
    v.y = *reinterpret_cast<const unsigned*>(&hi);
    *reinterpret_cast<uint2*>(p) = v;
  }
};
__device__ __forceinline__ float sum4(float4 a) { return (a.x + a.y) + (a.z + a.w); }
__device__ __forceinline__ float dev4(float4 a, float m) {
  const float x = a.x - m, y = a.y - m, z = a.z - m, w = a.w - m;
  return (x * x + y * y) + (z * z + w * w);
}
__device__ __forceinline__ float4 norm4(float4 a, float m, float inv, float4 w, float4 b) {
  return make_float4((a.x - m) * inv * w.x + b.x, (a.y - m) * inv * w.y + b.y, (a.z - m) * inv * w.z + b.z,
                     (a.w - m) * inv * w.w + b.w);
}

// The same with the row in registers: every input is asked for at once and read once, 16 bytes per access; RV pieces
// of four numbers per thread, for widths that are multiples of 4 up to 4 * RV * threads.
template <typename TA, typename TO, int RV, bool TWO>
__global__ void post_layer_norm_add_reg_kernel(float* __restrict__ x, const TA* __restrict__ a, const TA* __restrict__ b,
                                               float ca, float cb, const float* __restrict__ w,
                                               const float* __restrict__ bias, float mult,
                                               const float* __restrict__ w_next, const float* __restrict__ b_next,
                                               TO* __restrict__ out, const int* __restrict__ tok_seq, int width, float eps) {
  __shared__ float scratch[32];
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  const size_t row = (size_t)t * width;
  if (tok_seq != nullptr && tok_seq[t] < 0) {
    if (out != nullptr)
      for (int j = threadIdx.x; j < width; j += blockDim.x) out[row + j] = from_f32<TO>(0.f);
    return;
  }
  const float n = (float)width;
  float4 y[RV], xv[RV], wv[RV], bv[RV];
#pragma unroll
  for (int j = 0; j < RV; ++j) {
    const int i = (threadIdx.x + j * blockDim.x) * 4;
    if (i < width) {
      const float4 p = LnRow4<TA>::load(a + row + i);
      y[j] = make_float4(ca * p.x, ca * p.y, ca * p.z, ca * p.w);
      if (TWO) {
        const float4 q = LnRow4<TA>::load(b + row + i);
        y[j].x += cb * q.x;
        y[j].y += cb * q.y;
        y[j].z += cb * q.z;
        y[j].w += cb * q.w;
      }
      xv[j] = *reinterpret_cast<const float4*>(x + row + i);
      wv[j] = *reinterpret_cast<const float4*>(w + i);
      bv[j] = *reinterpret_cast<const float4*>(bias + i);
    }
  }
  float s = 0.f;
#pragma unroll
  for (int j = 0; j < RV; ++j)
    if ((threadIdx.x + j * blockDim.x) * 4 < width) s += sum4(y[j]);
  float mean = block_sum(s, scratch) / n;
  s = 0.f;
#pragma unroll
  for (int j = 0; j < RV; ++j)
    if ((threadIdx.x + j * blockDim.x) * 4 < width) s += dev4(y[j], mean);
  float inv = 1.0f / sqrtf(block_sum(s, scratch) / n + eps);
  s = 0.f;
#pragma unroll
  for (int j = 0; j < RV; ++j) {
    const int i = (threadIdx.x + j * blockDim.x) * 4;
    if (i < width) {
      const float4 d = norm4(y[j], mean, inv, wv[j], bv[j]);
      xv[j].x += mult * d.x;
      xv[j].y += mult * d.y;
      xv[j].z += mult * d.z;
      xv[j].w += mult * d.w;
      *reinterpret_cast<float4*>(x + row + i) = xv[j];
      s += sum4(xv[j]);
    }
  }
  if (out == nullptr) return;
#pragma unroll
  for (int j = 0; j < RV; ++j) {                 // the next norm's weight and bias take the places of this one's
    const int i = (threadIdx.x + j * blockDim.x) * 4;
    if (i < width) {
      wv[j] = *reinterpret_cast<const float4*>(w_next + i);
      bv[j] = *reinterpret_cast<const float4*>(b_next + i);
    }
  }
  mean = block_sum(s, scratch) / n;
  s = 0.f;
#pragma unroll
  for (int j = 0; j < RV; ++j)
    if ((threadIdx.x + j * blockDim.x) * 4 < width) s += dev4(xv[j], mean);
  inv = 1.0f / sqrtf(block_sum(s, scratch) / n + eps);
#pragma unroll
  for (int j = 0; j < RV; ++j) {
    const int i = (threadIdx.x + j * blockDim.x) * 4;
    if (i < width) LnRow4<TO>::store(out + row + i, norm4(xv[j], mean, inv, wv[j], bv[j]));
  }
}

AB_API int ab_post_layer_norm_add(float* x, const void* a, const void* b, int in_dtype, float ca, float cb, const float* w,
                                  const float* bias, float mult, const float* w_next, const float* b_next, void* out,
                                  int out_dtype, const int* tok_seq, int n_rows, int width, float eps,
                                  cudaStream_t stream) {
  if (n_rows <= 0 || width <= 0) return AB_OK;
  if (!x || !a || !w || !bias || (out && (!w_next || !b_next))) return AB_BAD_ARG;
  const size_t smem = (size_t)width * sizeof(float);
  if (smem > 200 * 1024) return AB_BAD_ARG;
  const int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
  const bool out_f32 = out == nullptr || out_dtype == AB_F32;
  if (!out_f32 && out_dtype != AB_BF16) return AB_BAD_ARG;
  if (in_dtype != AB_F32 && in_dtype != AB_BF16) return AB_BAD_ARG;
  const int vthreads = width >= 4096 ? 512 : (width >= 1024 ? 256 : 128);
  auto al = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
  if (width % 4 == 0 && width <= vthreads * 4 * 4 && al(x) && al(a) && al(b) && al(w) && al(bias) && al(w_next) &&
      al(b_next) && al(out)) {
#define AB_REG(TA, TO)                                                                                                    \
  {                                                                                                                       \
    if (b != nullptr)                                                                                                     \
      ab_launch(post_layer_norm_add_reg_kernel<TA, TO, 4, true>, dim3((unsigned)n_rows), dim3(vthreads), 0, stream, x,     \
                (const TA*)a, (const TA*)b, ca, cb, w, bias, mult, w_next, b_next, (TO*)out, tok_seq, width, eps);          \
    else                                                                                                                  \
      ab_launch(post_layer_norm_add_reg_kernel<TA, TO, 4, false>, dim3((unsigned)n_rows), dim3(vthreads), 0, stream, x,    \
                (const TA*)a, (const TA*)b, ca, cb, w, bias, mult, w_next, b_next, (TO*)out, tok_seq, width, eps);          \
  }
    if (in_dtype == AB_F32) { if (out_f32) AB_REG(float, float) else AB_REG(float, bf16) }
    else { if (out_f32) AB_REG(bf16, float) else AB_REG(bf16, bf16) }
#undef AB_REG
    return ab_launch_status();
  }
#define AB_GO(TA, TO)                                                                                                  \
  {                                                                                                                    \
    if (smem > 48 * 1024)                                                                                              \
      cudaFuncSetAttribute(post_layer_norm_add_kernel<TA, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    ab_launch(post_layer_norm_add_kernel<TA, TO>, dim3((unsigned)n_rows), dim3(threads), smem, stream, x, (const TA*)a, \
              (const TA*)b, ca, cb, w, bias, mult, w_next, b_next, (TO*)out, tok_seq, width, eps);                      \
  }
  if (in_dtype == AB_F32) { if (out_f32) AB_GO(float, float) else AB_GO(float, bf16) }
  else { if (out_f32) AB_GO(bf16, float) else AB_GO(bf16, bf16) }
#undef AB_GO
  return ab_launch_status();
}
