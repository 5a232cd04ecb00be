// Small kernels on the float32 residual stream that are not a norm before a sub-layer:
//
//   add_row        x[t, :] += row[:]                       a learned vector added to every token (a pass of a loop)
//   stream_cast    x += delta (if given); y = cast(x)      the stream itself as the input of a product
//   token_gate     a[t, j] = act(z[t, j]) * table[token_t, off + j]    a product gated by a per-token table row;
//                  act = gelu_tanh: 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))
//   add_unit_norm  x[t, :] += y[t, :] / sqrt(mean(y[t, :]^2) + eps) * w[:]
//   post_norm_add  the same for a sub-layer whose output is normed before it joins the stream, with the next
//                  sub-layer's norm in the same kernel:  y = a, or y = (unit(a) * wa + unit(b) * wb) / 2 for two
//                  sub-layers side by side;  x += unit(y) * w;  out = cast(unit(x) * w_next)  (if asked for);
//                  unit(v) = v / sqrt(mean(v^2) + eps)
//
// Arithmetic is 32-bit; rows whose sequence index is negative (padding of a captured step) are left alone by
// the kernels that write the stream.
#include "common.cuh"
#include "launch.cuh"

__global__ void add_row_kernel(float* __restrict__ x, const float* __restrict__ row, const int* __restrict__ tok_seq,
                               size_t total, int width) {
  pdl_wait();
  pdl_trigger();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const size_t t = i / width;
  if (tok_seq[t] < 0) return;
  x[i] += row[i - t * width];
}

template <typename T>
__global__ void stream_cast_kernel(float* __restrict__ x, const T* __restrict__ delta, T* __restrict__ y, size_t total) {
  pdl_wait();
  pdl_trigger();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  float v = x[i];
  if (delta != nullptr) {
    v += to_f32(delta[i]);
    x[i] = v;
  }
  y[i] = from_f32<T>(v);
}

__device__ __forceinline__ float gelu_tanh_f(float z) {
  return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

template <typename T>
__global__ void token_gate_kernel(const T* __restrict__ z, const T* __restrict__ table, int table_width, int off,
                                  const int* __restrict__ tokens, const int* __restrict__ tok_seq, T* __restrict__ out,
                                  size_t total, int dim) {
  pdl_wait();
  pdl_trigger();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const size_t t = i / dim;
  const int j = (int)(i - t * dim);
  if (tok_seq[t] < 0) { out[i] = from_f32<T>(0.f); return; }
  const float e = to_f32(table[(size_t)tokens[t] * table_width + off + j]);
  out[i] = from_f32<T>(gelu_tanh_f(to_f32(z[i])) * e);
}

// a block per row
__global__ void add_unit_norm_kernel(float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ w,
                                     const int* __restrict__ tok_seq, int width, float eps) {
  __shared__ float scratch[32];
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  if (tok_seq[t] < 0) return;
  const float* yr = y + (size_t)t * width;
  float ss = 0.f;
  for (int j = threadIdx.x; j < width; j += blockDim.x) ss += yr[j] * yr[j];
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)width + eps);
  float* xr = x + (size_t)t * width;
  for (int j = threadIdx.x; j < width; j += blockDim.x) xr[j] += yr[j] * inv * w[j];
}

// The same with the row in registers (one pass over memory, 16-byte accesses): 256 threads, NV pieces of four
// floats per thread, for widths that are multiples of 4 up to 1024 * NV.
template <int NV>
__global__ void __launch_bounds__(256)
add_unit_norm_vec_kernel(float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ w,
                         const int* __restrict__ tok_seq, int width, float eps) {
  __shared__ float scratch[32];
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  if (tok_seq[t] < 0) return;
  const int n4 = width >> 2;
  const float4* yr = reinterpret_cast<const float4*>(y + (size_t)t * width);
  float4* xr = reinterpret_cast<float4*>(x + (size_t)t * width);
  const float4* wr = reinterpret_cast<const float4*>(w);
  float4 yv[NV], xv[NV];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int i = threadIdx.x + k * 256;
    if (i < n4) {
      yv[k] = yr[i];
      xv[k] = xr[i];
      ss += (yv[k].x * yv[k].x + yv[k].y * yv[k].y) + (yv[k].z * yv[k].z + yv[k].w * yv[k].w);
    }
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)width + eps);
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int i = threadIdx.x + k * 256;
    if (i < n4) {
      const float4 wv = wr[i];
      xv[k].x += yv[k].x * inv * wv.x;
      xv[k].y += yv[k].y * inv * wv.y;
      xv[k].z += yv[k].z * inv * wv.z;
      xv[k].w += yv[k].w * inv * wv.w;
      xr[i] = xv[k];
    }
  }
}

// four elements per thread; delta and y bfloat16
__global__ void stream_cast_bf16x4_kernel(float* __restrict__ x, const bf16* __restrict__ delta, bf16* __restrict__ y,
                                          size_t n4) {
  pdl_wait();
  pdl_trigger();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n4) return;
  float4 v = reinterpret_cast<float4*>(x)[i];
  if (delta != nullptr) {
    const uint2 d = reinterpret_cast<const uint2*>(delta)[i];
    v.x += __uint_as_float(d.x << 16);
    v.y += __uint_as_float(d.x & 0xffff0000u);
    v.z += __uint_as_float(d.y << 16);
    v.w += __uint_as_float(d.y & 0xffff0000u);
    reinterpret_cast<float4*>(x)[i] = v;
  }
  __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
  reinterpret_cast<uint2*>(y)[i] = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
}

// four columns per thread (width a multiple of 4)
__global__ void add_row4_kernel(float* __restrict__ x, const float* __restrict__ row, const int* __restrict__ tok_seq,
                                size_t total4, int width4) {
  pdl_wait();
  pdl_trigger();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total4) return;
  const size_t t = i / width4;
  if (tok_seq[t] < 0) return;
  const float4 r = reinterpret_cast<const float4*>(row)[i - t * width4];
  float4 v = reinterpret_cast<float4*>(x)[i];
  v.x += r.x; v.y += r.y; v.z += r.z; v.w += r.w;
  reinterpret_cast<float4*>(x)[i] = v;
}

AB_API int ab_add_row(float* x, const float* row, const int* tok_seq, int n_rows, int width, cudaStream_t stream) {
  const size_t total = (size_t)n_rows * width;
  if (total == 0) return AB_OK;
  if (width % 4 == 0 && (reinterpret_cast<uintptr_t>(row) & 15) == 0) {
    ab_launch(add_row4_kernel, dim3((unsigned)((total / 4 + 255) / 256)), dim3(256), 0, stream, x, row, tok_seq, total / 4,
              width / 4);
    return ab_launch_status();
  }
  ab_launch(add_row_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, x, row, tok_seq, total, width);
  return ab_launch_status();
}

AB_API int ab_stream_cast(float* x, const void* delta, void* y, int dtype, int n_rows, int width, cudaStream_t stream) {
  const size_t total = (size_t)n_rows * width;
  if (total == 0) return AB_OK;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (dtype == AB_F32)
    ab_launch(stream_cast_kernel<float>, dim3(blocks), dim3(256), 0, stream, x, (const float*)delta, (float*)y, total);
  else if (dtype == AB_BF16 && width % 4 == 0)
    ab_launch(stream_cast_bf16x4_kernel, dim3((unsigned)((total / 4 + 255) / 256)), dim3(256), 0, stream, x,
              (const bf16*)delta, (bf16*)y, total / 4);
  else if (dtype == AB_BF16)
    ab_launch(stream_cast_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, x, (const bf16*)delta, (bf16*)y, total);
  else
    return AB_BAD_ARG;
  return ab_launch_status();
}

AB_API int ab_token_gate(const void* z, const void* table, int table_width, int off, const int* tokens,
                         const int* tok_seq, void* out, int dtype, int n_rows, int dim, cudaStream_t stream) {
  const size_t total = (size_t)n_rows * dim;
  if (total == 0) return AB_OK;
  if (off < 0 || off + dim > table_width) return AB_BAD_ARG;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (dtype == AB_F32)
    ab_launch(token_gate_kernel<float>, dim3(blocks), dim3(256), 0, stream, (const float*)z, (const float*)table,
              table_width, off, tokens, tok_seq, (float*)out, total, dim);
  else if (dtype == AB_BF16)
    ab_launch(token_gate_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, (const bf16*)z, (const bf16*)table,
              table_width, off, tokens, tok_seq, (bf16*)out, total, dim);
  else
    return AB_BAD_ARG;
  return ab_launch_status();
}

AB_API int ab_add_unit_norm(float* x, const float* y, const float* w, const int* tok_seq, int n_rows, int width, float eps,
                            cudaStream_t stream) {
  if (n_rows <= 0 || width <= 0) return AB_OK;
  if (width % 4 == 0 && width <= 8192) {
#define AB_GO(NV) ab_launch(add_unit_norm_vec_kernel<NV>, dim3((unsigned)n_rows), dim3(256), 0, stream, x, y, w, tok_seq, width, eps)
    if (width <= 1024) AB_GO(1);
    else if (width <= 2048) AB_GO(2);
    else if (width <= 4096) AB_GO(4);
    else AB_GO(8);
#undef AB_GO
    return ab_launch_status();
  }
  const int threads = width >= 2048 ? 256 : 128;
  ab_launch(add_unit_norm_kernel, dim3((unsigned)n_rows), dim3(threads), 0, stream, x, y, w, tok_seq, width, eps);
  return ab_launch_status();
}


// A block per row; the row of y waits in shared memory between the passes (width floats).  TA: the dtype of a and b.
template <typename TA, typename TO>
__global__ void __launch_bounds__(256)
post_norm_add_kernel(float* __restrict__ x, const TA* __restrict__ a, const TA* __restrict__ b,
                     const float* __restrict__ wa, const float* __restrict__ wb, const float* __restrict__ w,
                     const float* __restrict__ w_next, TO* __restrict__ out, const int* __restrict__ tok_seq, int width,
                     float eps) {
  extern __shared__ float pn_row[];
  __shared__ float scratch[32];
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  if (tok_seq != nullptr && tok_seq[t] < 0) {
    if (out != nullptr)
      for (int j = threadIdx.x; j < width; j += blockDim.x) out[(size_t)t * width + j] = from_f32<TO>(0.f);
    return;
  }
  const TA* ar = a + (size_t)t * width;
  const float n = (float)width;
  float sa = 0.f, sb = 0.f;
  if (b == nullptr) {
    for (int j = threadIdx.x; j < width; j += blockDim.x) {
      const float v = to_f32(ar[j]);
      pn_row[j] = v;
      sa += v * v;
    }
    sa = block_sum(sa, scratch);
  } else {
    const TA* br = b + (size_t)t * width;
    for (int j = threadIdx.x; j < width; j += blockDim.x) {
      const float u = to_f32(ar[j]), v = to_f32(br[j]);
      sa += u * u;
      sb += v * v;
    }
    sa = block_sum(sa, scratch);
    sb = block_sum(sb, scratch);
    const float ia = 1.0f / sqrtf(sa / n + eps), ib = 1.0f / sqrtf(sb / n + eps);
    sa = 0.f;
    for (int j = threadIdx.x; j < width; j += blockDim.x) {
      const float v = 0.5f * (to_f32(ar[j]) * ia * wa[j] + to_f32(br[j]) * ib * wb[j]);
      pn_row[j] = v;
      sa += v * v;
    }
    sa = block_sum(sa, scratch);
  }
  const float inv = 1.0f / sqrtf(sa / n + eps);
  float* xr = x + (size_t)t * width;
  float sx = 0.f;
  for (int j = threadIdx.x; j < width; j += blockDim.x) {      // a thread meets its own elements of the row again
    const float v = xr[j] + pn_row[j] * inv * w[j];
    xr[j] = v;
    pn_row[j] = v;
    sx += v * v;
  }
  if (out == nullptr) return;
  sx = block_sum(sx, scratch);
  const float ix = 1.0f / sqrtf(sx / n + eps);
  TO* o = out + (size_t)t * width;
  for (int j = threadIdx.x; j < width; j += blockDim.x) o[j] = from_f32<TO>(pn_row[j] * ix * w_next[j]);
}

// Four numbers of a row per access (widths that are multiples of 4).
template <typename T> struct Row4;
template <> struct Row4<float> {
  float4 v;
  __device__ __forceinline__ void load(const float* p) { v = *reinterpret_cast<const float4*>(p); }
  __device__ __forceinline__ void store(float* p) const { *reinterpret_cast<float4*>(p) = v; }
  __device__ __forceinline__ float4 get() const { return v; }
  __device__ __forceinline__ void set(float4 a) { v = a; }
};
template <> struct Row4<bf16> {
  uint2 v;
  __device__ __forceinline__ void load(const bf16* p) { v = *reinterpret_cast<const uint2*>(p); }
  __device__ __forceinline__ void store(bf16* p) const { *reinterpret_cast<uint2*>(p) = v; }
  __device__ __forceinline__ float4 get() const {
    return make_float4(__uint_as_float(v.x << 16), __uint_as_float(v.x & 0xffff0000u), __uint_as_float(v.y << 16),
                       __uint_as_float(v.y & 0xffff0000u));
  }
  __device__ __forceinline__ void set(float4 a) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a.x, a.y), hi = __floats2bfloat162_rn(a.z, a.w);
    v.x = *reinterpret_cast<uint32_t*>(&lo);
    v.y = *reinterpret_cast<uint32_t*>(&hi);
  }
};
__device__ __forceinline__ float sq4(float4 v) { return v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w; }

// The same for rows short enough that a thread keeps its share in registers (up to RV x 4 numbers per thread): the
// sub-layer's outputs, the stream's row and every weight are asked for at once and read once.  TWO: two inputs.
template <typename TA, typename TO, int RV, bool TWO>
__global__ void __launch_bounds__(512)
post_norm_add_reg_kernel(float* __restrict__ x, const TA* __restrict__ a, const TA* __restrict__ b,
                         const float* __restrict__ wa, const float* __restrict__ wb, const float* __restrict__ w,
                         const float* __restrict__ w_next, TO* __restrict__ out, const int* __restrict__ tok_seq,
                         int width, float eps) {
  __shared__ float scratch[32];
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  if (tok_seq != nullptr && tok_seq[t] < 0) {
    if (out != nullptr)
      for (int j = threadIdx.x; j < width; j += blockDim.x) out[(size_t)t * width + j] = from_f32<TO>(0.f);
    return;
  }
  const size_t row = (size_t)t * width;
  const float n = (float)width;
  float4 y[RV], xv[RV], wv[RV], wn[RV], wav[RV], wbv[RV], bv[RV];
#pragma unroll
  for (int j = 0; j < RV; ++j) {
    const int i = (threadIdx.x + j * blockDim.x) * 4;
    if (i < width) {
      Row4<TA> r;
      r.load(a + row + i);
      y[j] = r.get();
      if (TWO) {
        r.load(b + row + i);
        bv[j] = r.get();
        wav[j] = *reinterpret_cast<const float4*>(wa + i);
        wbv[j] = *reinterpret_cast<const float4*>(wb + i);
      }
      xv[j] = *reinterpret_cast<const float4*>(x + row + i);
      wv[j] = *reinterpret_cast<const float4*>(w + i);
      if (out != nullptr) wn[j] = *reinterpret_cast<const float4*>(w_next + i);
    }
  }
  float sa = 0.f, sb = 0.f;
#pragma unroll
  for (int j = 0; j < RV; ++j)
    if ((threadIdx.x + j * blockDim.x) * 4 < width) {
      sa += sq4(y[j]);
      if (TWO) sb += sq4(bv[j]);
    }
  sa = block_sum(sa, scratch);
  if (TWO) {
    sb = block_sum(sb, scratch);
    const float ia = 1.0f / sqrtf(sa / n + eps), ib = 1.0f / sqrtf(sb / n + eps);
    sa = 0.f;
#pragma unroll
    for (int j = 0; j < RV; ++j)
      if ((threadIdx.x + j * blockDim.x) * 4 < width) {
        y[j].x = 0.5f * (y[j].x * ia * wav[j].x + bv[j].x * ib * wbv[j].x);
        y[j].y = 0.5f * (y[j].y * ia * wav[j].y + bv[j].y * ib * wbv[j].y);
        y[j].z = 0.5f * (y[j].z * ia * wav[j].z + bv[j].z * ib * wbv[j].z);
        y[j].w = 0.5f * (y[j].w * ia * wav[j].w + bv[j].w * ib * wbv[j].w);
        sa += sq4(y[j]);
      }
    sa = block_sum(sa, scratch);
  }
  const float inv = 1.0f / sqrtf(sa / n + eps);
  float sx = 0.f;
#pragma unroll
  for (int j = 0; j < RV; ++j) {
    const int i = (threadIdx.x + j * blockDim.x) * 4;
    if (i < width) {
      xv[j].x += y[j].x * inv * wv[j].x;
      xv[j].y += y[j].y * inv * wv[j].y;
      xv[j].z += y[j].z * inv * wv[j].z;
      xv[j].w += y[j].w * inv * wv[j].w;
      *reinterpret_cast<float4*>(x + row + i) = xv[j];
      sx += sq4(xv[j]);
    }
  }
  if (out == nullptr) return;
  sx = block_sum(sx, scratch);
  const float ix = 1.0f / sqrtf(sx / n + eps);
#pragma unroll
  for (int j = 0; j < RV; ++j) {
    const int i = (threadIdx.x + j * blockDim.x) * 4;
    if (i < width) {
      Row4<TO> o;
      o.set(make_float4(xv[j].x * ix * wn[j].x, xv[j].y * ix * wn[j].y, xv[j].z * ix * wn[j].z, xv[j].w * ix * wn[j].w));
      o.store(out + row + i);
    }
  }
}

// a, b: [n_rows, width] of dtype `in_dtype` (b, wa, wb null: one input); out of dtype `out_dtype` or null.
AB_API int ab_post_norm_add(float* x, const void* a, const void* b, int in_dtype, const float* wa, const float* wb,
                            const float* w, const float* w_next, void* out, int out_dtype, const int* tok_seq, int n_rows,
                            int width, float eps, cudaStream_t stream) {
  if (n_rows <= 0 || width <= 0) return AB_OK;
  if (!x || !a || !w || (b && (!wa || !wb)) || (out && !w_next)) return AB_BAD_ARG;
  const bool out_f32 = out == nullptr || out_dtype == AB_F32;
  if (!out_f32 && out_dtype != AB_BF16) return AB_BAD_ARG;
  if (in_dtype != AB_F32 && in_dtype != AB_BF16) return AB_BAD_ARG;
  const int vthreads = width >= 4096 ? 512 : (width >= 1024 ? 256 : 128);
  if (width % 4 == 0 && width <= vthreads * 4 * 4) {
#define AB_REG(TA, TO)                                                                                               \
  {                                                                                                                  \
    if (b != nullptr)                                                                                                \
      ab_launch(post_norm_add_reg_kernel<TA, TO, 4, true>, dim3((unsigned)n_rows), dim3(vthreads), 0, stream, x,     \
                (const TA*)a, (const TA*)b, wa, wb, w, w_next, (TO*)out, tok_seq, width, eps);                       \
    else                                                                                                             \
      ab_launch(post_norm_add_reg_kernel<TA, TO, 4, false>, dim3((unsigned)n_rows), dim3(vthreads), 0, stream, x,    \
                (const TA*)a, (const TA*)b, wa, wb, w, w_next, (TO*)out, tok_seq, width, eps);                       \
  }
    if (in_dtype == AB_F32) { if (out_f32) AB_REG(float, float) else AB_REG(float, bf16) }
    else { if (out_f32) AB_REG(bf16, float) else AB_REG(bf16, bf16) }
#undef AB_REG
    return ab_launch_status();
  }
  const size_t smem = (size_t)width * sizeof(float);
  if (smem > 200 * 1024) return AB_BAD_ARG;
  const int threads = width >= 1024 ? 256 : 128;
#define AB_GO(TA, TO)                                                                                                   \
  {                                                                                                                     \
    if (smem > 48 * 1024) {                                                                                             \
      cudaError_t e = cudaFuncSetAttribute(post_norm_add_kernel<TA, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize,   \
                                           (int)smem);                                                                  \
      if (e != cudaSuccess) return AB_CUDA_ERR + (int)e;                                                                \
    }                                                                                                                   \
    ab_launch(post_norm_add_kernel<TA, TO>, dim3((unsigned)n_rows), dim3(threads), smem, stream, x, (const TA*)a,       \
              (const TA*)b, wa, wb, w, w_next, (TO*)out, tok_seq, width, eps);                                          \
  }
  if (in_dtype == AB_F32) { if (out_f32) AB_GO(float, float) else AB_GO(float, bf16) }
  else if (in_dtype == AB_BF16) { if (out_f32) AB_GO(bf16, float) else AB_GO(bf16, bf16) }
  else return AB_BAD_ARG;
#undef AB_GO
  return ab_launch_status();
}

// ---------------------------------------------------------------------------------------------
// embed_pairs: the stream's first value for a model whose embedding has a factor and a hashed table of (previous
// token, token) pairs:  x[t] = table[token_t] * scale + pairs[(prev_t * mul_prev + token_t * mul_cur) mod buckets],
// and row `buckets` (the last one) of `pairs` for a sequence's first token.  The previous token of a step's first
// token is what the sequence keeps from its last step: `last_token[slot]`, which the block of that first token
// reads and then sets to the step's last token of the sequence (one thread does both, in this order).
// A block per token; rows without a sequence become zero.
template <typename T>
__global__ void embed_pairs_kernel(const T* __restrict__ table, float scale, const T* __restrict__ pairs, long long buckets,
                                   long long mul_prev, long long mul_cur, const int* __restrict__ tokens,
                                   const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                                   const int* __restrict__ cu_q, const int* __restrict__ slots,
                                   int* __restrict__ last_token, float* __restrict__ out, int width) {
  __shared__ long long pair_row;
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  const int b = tok_seq[t];
  float* o = out + (size_t)t * width;
  if (b < 0) {
    for (int j = threadIdx.x; j < width; j += blockDim.x) o[j] = 0.f;
    return;
  }
  const int tok = tokens[t];
  if (pairs != nullptr) {
    if (threadIdx.x == 0) {
      const int first = cu_q[b];
      long long row = buckets;
      if (tok_pos[t] > 0) {
        const long long prev = t > first ? tokens[t - 1] : last_token[slots[b]];
        row = (prev * mul_prev + (long long)tok * mul_cur) % buckets;
      }
      if (t == first) last_token[slots[b]] = tokens[cu_q[b + 1] - 1];
      pair_row = row;
    }
    __syncthreads();
  }
  const T* e = table + (size_t)tok * width;
  if (pairs == nullptr) {
    for (int j = threadIdx.x; j < width; j += blockDim.x) o[j] = to_f32(e[j]) * scale;
    return;
  }
  const T* p = pairs + (size_t)pair_row * width;
  for (int j = threadIdx.x; j < width; j += blockDim.x) o[j] = to_f32(e[j]) * scale + to_f32(p[j]);
}

AB_API int ab_embed_pairs(const void* table, int dtype, float scale, const void* pairs, long long buckets,
                          long long mul_prev, long long mul_cur, const int* tokens, const int* tok_seq, const int* tok_pos,
                          const int* cu_q, const int* slots, int* last_token, float* out, int n_tokens, int width,
                          cudaStream_t stream) {
  if (n_tokens <= 0 || width <= 0) return AB_OK;
  if (!table || !tokens || !tok_seq || !out) return AB_BAD_ARG;
  if (pairs && (!tok_pos || !cu_q || !slots || !last_token || buckets <= 0 || mul_prev < 0 || mul_cur < 0)) return AB_BAD_ARG;
  const int threads = width >= 1024 ? 256 : 128;
  if (dtype == AB_F32)
    ab_launch(embed_pairs_kernel<float>, dim3((unsigned)n_tokens), dim3(threads), 0, stream, (const float*)table, scale,
              (const float*)pairs, buckets, mul_prev, mul_cur, tokens, tok_seq, tok_pos, cu_q, slots, last_token, out, width);
  else if (dtype == AB_BF16)
    ab_launch(embed_pairs_kernel<bf16>, dim3((unsigned)n_tokens), dim3(threads), 0, stream, (const bf16*)table, scale,
              (const bf16*)pairs, buckets, mul_prev, mul_cur, tokens, tok_seq, tok_pos, cu_q, slots, last_token, out, width);
  else
    return AB_BAD_ARG;
  return ab_launch_status();
}

// head_gate: y[t, h, :] *= sigmoid(g[t * g_stride + h]): one gate per head and token, 32-bit arithmetic
template <typename T, typename TG>
__global__ void head_gate_kernel(T* __restrict__ y, const TG* __restrict__ g, int g_stride, size_t total, int H, int V) {
  pdl_wait();
  pdl_trigger();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const size_t th = i / V;
  const size_t t = th / H;
  const float z = to_f32(g[t * g_stride + (th - t * H)]);
  y[i] = from_f32<T>(to_f32(y[i]) / (1.0f + expf(-z)));
}

AB_API int ab_head_gate(void* y, int dtype, const void* g, int g_dtype, int g_stride, int n_tokens, int H, int V,
                        cudaStream_t stream) {
  if (n_tokens <= 0 || H <= 0 || V <= 0) return AB_OK;
  if (!y || !g || g_stride < H) return AB_BAD_ARG;
  const size_t total = (size_t)n_tokens * H * V;
  const unsigned blocks = (unsigned)((total + 255) / 256);
#define AB_GO(T, TG) ab_launch(head_gate_kernel<T, TG>, dim3(blocks), dim3(256), 0, stream, (T*)y, (const TG*)g, g_stride, total, H, V)
  if (dtype == AB_F32 && g_dtype == AB_F32) AB_GO(float, float);
  else if (dtype == AB_BF16 && g_dtype == AB_BF16) AB_GO(bf16, bf16);
  else if (dtype == AB_BF16 && g_dtype == AB_F32) AB_GO(bf16, float);
  else if (dtype == AB_F32 && g_dtype == AB_BF16) AB_GO(float, bf16);
  else return AB_BAD_ARG;
#undef AB_GO
  return ab_launch_status();
}
