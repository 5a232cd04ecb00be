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
// A block per row; the row waits in shared memory between the passes (mean, then squared deviations, then the
// result: the variance is taken about the mean, not as a difference of two sums).  Arithmetic is 32-bit; rows
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
