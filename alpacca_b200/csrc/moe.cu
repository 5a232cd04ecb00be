// Routed experts: the router with groups, and the experts' two products for the (token, expert) pairs of a step.
//
// Router, per token, in 32-bit: z = W_r h; s = softmax(z) over all experts; the experts form `groups` equal
// groups of neighbours, a group's score is its largest s, only experts of the `keep` best groups can be
// chosen; the `top` largest s among those are chosen (the lower index wins a tie); their weights are
// s / (sum of the chosen s + 1e-20) * scale.
// Experts: y_t = sum_j weight_j * W_down[e_j] act(W_up[e_j] h_t), act = exact gelu (erf) here.
// Options: a bias on the router's logits; gated experts, y_t = sum_j weight_j * W_down[e_j] (act(W_gate[e_j] h_t) *
// (W_up[e_j] h_t)).  (With one group, all groups kept and scale 1 the weights are the softmax over the chosen
// logits alone: s_j / sum of the chosen s is exp(z_j) / sum of the chosen exp(z).)
// The pair kernels read each chosen expert's rows once per pair: the form for steps of few tokens, where the
// weights stream from memory once and every token adds its experts in the order of its choices.
#include "common.cuh"
#include "launch.cuh"

#define MOE_MAX_EXPERTS 1024

// A warp's share of the dot product of two rows of n numbers (add with warp_sum): 16 bytes per lane and
// load where both rows allow it.
__device__ __forceinline__ float lane_dot(const bf16* __restrict__ a, const bf16* __restrict__ b, int n, int lane) {
  float part = 0.f;
  if ((n & 7) == 0 && ((((uintptr_t)a) | ((uintptr_t)b)) & 15) == 0) {
    for (int k = lane * 8; k < n; k += 256) {
      const uint4 x = *reinterpret_cast<const uint4*>(a + k);
      const uint4 y = __ldg(reinterpret_cast<const uint4*>(b + k));
      const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(&x);
      const __nv_bfloat162* yp = reinterpret_cast<const __nv_bfloat162*>(&y);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 xf = __bfloat1622float2(xp[j]), yf = __bfloat1622float2(yp[j]);
        part += xf.x * yf.x + xf.y * yf.y;
      }
    }
    return part;
  }
  for (int k = lane; k < n; k += 32) part += __bfloat162float(a[k]) * __bfloat162float(b[k]);
  return part;
}
__device__ __forceinline__ float lane_dot(const float* __restrict__ a, const float* __restrict__ b, int n, int lane) {
  float part = 0.f;
  for (int k = lane; k < n; k += 32) part += a[k] * b[k];      // one order for every n: the 32-bit path
  return part;
}
__device__ __forceinline__ float lane_dot(const bf16* __restrict__ a, const float* __restrict__ b, int n, int lane) {
  float part = 0.f;
  if ((n & 3) == 0 && (((uintptr_t)a) & 7) == 0 && (((uintptr_t)b) & 15) == 0) {
    for (int k = lane * 4; k < n; k += 128) {
      const uint2 x = *reinterpret_cast<const uint2*>(a + k);
      const float4 y = __ldg(reinterpret_cast<const float4*>(b + k));
      const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(&x);
      const float2 x0 = __bfloat1622float2(xp[0]), x1 = __bfloat1622float2(xp[1]);
      part += x0.x * y.x + x0.y * y.y + x1.x * y.z + x1.y * y.w;
    }
    return part;
  }
  for (int k = lane; k < n; k += 32) part += __bfloat162float(a[k]) * b[k];
  return part;
}

// z[t, e] = W_r[e] . h[t]: one warp per (token, expert)
template <typename T>
__global__ void moe_logits_kernel(const T* __restrict__ h, int ld, const float* __restrict__ wr, int n_tokens, int width,
                                  int E, float* __restrict__ z, const float* __restrict__ bias) {
  pdl_wait();
  pdl_trigger();
  const int lane = threadIdx.x & 31;
  const long long id = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (id >= (long long)n_tokens * E) return;
  const int t = (int)(id / E), e = (int)(id - (long long)t * E);
  const float part = warp_sum(lane_dot(h + (size_t)t * ld, wr + (size_t)e * width, width, lane));
  if (lane == 0) z[id] = part + (bias != nullptr ? bias[e] : 0.f);
}

// the choice, one warp per token, from the logits z [T, E]
__global__ void moe_route_kernel(const float* __restrict__ z, int n_tokens, int E, int groups, int keep, int top,
                                 float scale, int* __restrict__ idx, float* __restrict__ wts) {
  extern __shared__ float sm[];           // E scores per warp, then `groups` group scores per warp
  pdl_wait();
  pdl_trigger();
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  const int t = blockIdx.x * (blockDim.x >> 5) + wib;
  if (t >= n_tokens) return;
  float* s = sm + (size_t)wib * E;
  for (int e = lane; e < E; e += 32) s[e] = z[(size_t)t * E + e];
  __syncwarp();
  float mx = -INFINITY;
  for (int e = lane; e < E; e += 32) mx = fmaxf(mx, s[e]);
  mx = warp_max(mx);
  float sum = 0.f;
  for (int e = lane; e < E; e += 32) {
    const float p = expf(s[e] - mx);
    s[e] = p;
    sum += p;
  }
  sum = warp_sum(sum);
  __syncwarp();
  for (int e = lane; e < E; e += 32) s[e] = s[e] / sum;
  __syncwarp();
  // groups: the experts of groups that are not kept are struck out (-1, below every score)
  const int per = E / groups;
  if (keep < groups) {
    float* gs = sm + (size_t)(blockDim.x >> 5) * E + (size_t)wib * groups;
    for (int g = lane; g < groups; g += 32) {
      float v = -1.f;
      for (int j = 0; j < per; ++j) v = fmaxf(v, s[g * per + j]);
      gs[g] = v;
    }
    __syncwarp();
    for (int pick = 0; pick < keep; ++pick) {
      float best = -0.5f;
      int bg = 0x7fffffff;
      for (int g = lane; g < groups; g += 32)
        if (gs[g] > best) { best = gs[g]; bg = g; }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int og = __shfl_xor_sync(0xffffffffu, bg, o);
        if (ob > best || (ob == best && og < bg)) { best = ob; bg = og; }
      }
      if (lane == 0 && bg != 0x7fffffff) gs[bg] = -2.f;      // kept
      __syncwarp();
    }
    for (int e = lane; e < E; e += 32)
      if (gs[e / per] != -2.f) s[e] = -1.f;
    __syncwarp();
  }
  float chosen_sum = 0.f;
  for (int pick = 0; pick < top; ++pick) {
    float best = -0.5f;
    int be = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float v = s[e];
      if (v > best) { best = v; be = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, be, o);
      if (ob > best || (ob == best && oe < be)) { best = ob; be = oe; }
    }
    if (be == 0x7fffffff) { be = 0; best = 0.f; }      // nothing left to choose (or the row holds no numbers)
    chosen_sum += best;
    if (lane == 0) {
      idx[(size_t)t * top + pick] = be;
      wts[(size_t)t * top + pick] = best;
      s[be] = -1.f;                                    // taken
    }
    __syncwarp();
  }
  if (lane == 0) {
    const float inv = scale / (chosen_sum + 1e-20f);
    for (int j = 0; j < top; ++j) wts[(size_t)t * top + j] *= inv;
  }
}

// `bias`: float [E] added to the logits, or null
AB_API int ab_moe_route_bias(const void* h, int dtype, int ld, const float* wr, const float* bias, int n_tokens, int width,
                             int E, int groups, int keep, int top, float scale, float* z, int* idx, float* wts,
                             cudaStream_t stream) {
  if (n_tokens <= 0) return AB_OK;
  if (E <= 0 || E > MOE_MAX_EXPERTS || groups <= 0 || E % groups || keep <= 0 || keep > groups || top <= 0 ||
      top > keep * (E / groups))
    return AB_BAD_ARG;
  const int wpb = 4;
  const long long lw = (long long)n_tokens * E;
  const unsigned lblocks = (unsigned)((lw + 7) / 8);
  if (dtype == AB_F32)
    ab_launch(moe_logits_kernel<float>, dim3(lblocks), dim3(256), 0, stream, (const float*)h, ld, wr, n_tokens, width, E, z, bias);
  else if (dtype == AB_BF16)
    ab_launch(moe_logits_kernel<bf16>, dim3(lblocks), dim3(256), 0, stream, (const bf16*)h, ld, wr, n_tokens, width, E, z, bias);
  else
    return AB_BAD_ARG;
  int rc = ab_launch_status();
  if (rc) return rc;
  const unsigned blocks = (unsigned)((n_tokens + wpb - 1) / wpb);
  const size_t smem = (size_t)wpb * (E + groups) * sizeof(float);
  ab_launch(moe_route_kernel, dim3(blocks), dim3(wpb * 32), smem, stream, (const float*)z, n_tokens, E, groups, keep, top,
            scale, idx, wts);
  return ab_launch_status();
}

AB_API int ab_moe_route(const void* h, int dtype, int ld, const float* wr, int n_tokens, int width, int E, int groups,
                        int keep, int top, float scale, float* z, int* idx, float* wts, cudaStream_t stream) {
  return ab_moe_route_bias(h, dtype, ld, wr, nullptr, n_tokens, width, E, groups, keep, top, scale, z, idx, wts, stream);
}

// The choice from scores that are not a softmax, one warp per token, from the logits z [T, E]:
//   s = sigmoid(z) (score_fn 1) or z itself (0);  the CHOICE is made by c = s + correction (if given), the weights
//   are the chosen experts' s, times `scale`, divided by their sum if `renorm`.
//   Groups: a group's score is the sum of its `group_top` largest c; experts outside the `keep` best groups cannot be
//   chosen whatever their c (choice scores may be negative, so they are struck out with minus infinity).
// The lower index wins a tie, among groups and among experts.
__global__ void moe_route_scores_kernel(const float* __restrict__ z, const float* __restrict__ correction, int n_tokens,
                                        int E, int groups, int keep, int group_top, int top, int score_fn, int renorm,
                                        float scale, int* __restrict__ idx, float* __restrict__ wts) {
  extern __shared__ float sm[];           // per warp: E scores, E choice scores, `groups` group scores
  pdl_wait();
  pdl_trigger();
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  const int t = blockIdx.x * (blockDim.x >> 5) + wib;
  if (t >= n_tokens) return;
  float* s = sm + (size_t)wib * (2 * E + groups);
  float* c = s + E;
  float* gs = c + E;
  for (int e = lane; e < E; e += 32) {
    const float v = z[(size_t)t * E + e];
    const float sc = score_fn == 1 ? 1.0f / (1.0f + expf(-v)) : v;
    s[e] = sc;
    c[e] = sc + (correction != nullptr ? correction[e] : 0.f);
  }
  __syncwarp();
  const int per = E / groups;
  if (keep < groups) {
    for (int g = lane; g < groups; g += 32) {
      // the sum of the group's `group_top` largest choice scores, by repeated arg-max over a few members
      float total = 0.f;
      unsigned long long taken_lo = 0, taken_hi = 0;      // members already counted (a group of up to 128)
      for (int pick = 0; pick < group_top && pick < per; ++pick) {
        float best = -INFINITY;
        int bj = -1;
        for (int j = 0; j < per; ++j) {
          const bool used = j < 64 ? (taken_lo >> j) & 1ull : (taken_hi >> (j - 64)) & 1ull;
          if (!used && (bj < 0 || c[g * per + j] > best)) { best = c[g * per + j]; bj = j; }
        }
        if (bj < 64) taken_lo |= 1ull << bj; else taken_hi |= 1ull << (bj - 64);
        total += best;
      }
      gs[g] = total;
    }
    __syncwarp();
    for (int pick = 0; pick < keep; ++pick) {
      float best = -INFINITY;
      int bg = 0x7fffffff;
      for (int g = lane; g < groups; g += 32)
        if (!isnan(gs[g]) && (bg == 0x7fffffff || gs[g] > best)) { best = gs[g]; bg = g; }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int og = __shfl_xor_sync(0xffffffffu, bg, o);
        if (og != 0x7fffffff && (bg == 0x7fffffff || ob > best || (ob == best && og < bg))) { best = ob; bg = og; }
      }
      if (lane == 0 && bg != 0x7fffffff) gs[bg] = __int_as_float(0x7fc00000);      // kept: marked with a NaN
      __syncwarp();
    }
    for (int e = lane; e < E; e += 32)
      if (!isnan(gs[e / per])) c[e] = -INFINITY;
    __syncwarp();
  }
  float chosen_sum = 0.f;
  for (int pick = 0; pick < top; ++pick) {
    float best = -INFINITY;
    int be = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float v = c[e];
      if (v > best) { best = v; be = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, be, o);
      if (ob > best || (ob == best && oe < be)) { best = ob; be = oe; }
    }
    if (be == 0x7fffffff) be = 0;                      // nothing left to choose (or the row holds no numbers)
    const float w = s[be];
    chosen_sum += w;
    if (lane == 0) {
      idx[(size_t)t * top + pick] = be;
      wts[(size_t)t * top + pick] = w;
    }
    __syncwarp();
    if (lane == 0) c[be] = -INFINITY;                  // taken
    __syncwarp();
  }
  if (lane == 0) {
    const float f = renorm ? scale / (chosen_sum + 1e-20f) : scale;
    for (int j = 0; j < top; ++j) wts[(size_t)t * top + j] *= f;
  }
}

AB_API int ab_moe_route_scores(const void* h, int dtype, int ld, const float* wr, const float* bias, const float* correction,
                               int n_tokens, int width, int E, int groups, int keep, int group_top, int top, int score_fn,
                               int renorm, float scale, float* z, int* idx, float* wts, cudaStream_t stream) {
  if (n_tokens <= 0) return AB_OK;
  if (E <= 0 || E > MOE_MAX_EXPERTS || groups <= 0 || E % groups || keep <= 0 || keep > groups || top <= 0 ||
      top > keep * (E / groups) || group_top <= 0 || E / groups > 128 || score_fn < 0 || score_fn > 1)
    return AB_BAD_ARG;
  const int wpb = 4;
  const long long lw = (long long)n_tokens * E;
  const unsigned lblocks = (unsigned)((lw + 7) / 8);
  if (dtype == AB_F32)
    ab_launch(moe_logits_kernel<float>, dim3(lblocks), dim3(256), 0, stream, (const float*)h, ld, wr, n_tokens, width, E, z, bias);
  else if (dtype == AB_BF16)
    ab_launch(moe_logits_kernel<bf16>, dim3(lblocks), dim3(256), 0, stream, (const bf16*)h, ld, wr, n_tokens, width, E, z, bias);
  else
    return AB_BAD_ARG;
  int rc = ab_launch_status();
  if (rc) return rc;
  const unsigned blocks = (unsigned)((n_tokens + wpb - 1) / wpb);
  const size_t smem = (size_t)wpb * (2 * E + groups) * sizeof(float);
  ab_launch(moe_route_scores_kernel, dim3(blocks), dim3(wpb * 32), smem, stream, (const float*)z, correction, n_tokens, E,
            groups, keep, group_top, top, score_fn, renorm, scale, idx, wts);
  return ab_launch_status();
}

__device__ __forceinline__ float gelu_erf(float z) { return 0.5f * z * (1.0f + erff(z * 0.70710678118654752440f)); }
__device__ __forceinline__ float silu(float z) { return z / (1.0f + expf(-z)); }

// act[p, j] = f(W_up[e_p][j] . h[t_p]) for pair p = t * top + k, or, gated (w_gate given),
// f(W_gate[e_p][j] . h[t_p]) * (W_up[e_p][j] . h[t_p]).  One warp per (pair, j).
template <typename T>
__global__ void moe_up_pairs_kernel(const T* __restrict__ h, int ld, const T* __restrict__ w_up, const T* __restrict__ w_gate,
                                    const int* __restrict__ idx, T* __restrict__ act, int n_pairs, int top, int width,
                                    int ff, int activation) {
  pdl_wait();
  pdl_trigger();
  const int lane = threadIdx.x & 31;
  const long long id = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (id >= (long long)n_pairs * ff) return;
  const int p = (int)(id / ff), j = (int)(id - (long long)p * ff);
  const int e = idx[p];
  const T* x = h + (size_t)(p / top) * ld;
  const float part = warp_sum(lane_dot(x, w_up + ((size_t)e * ff + j) * width, width, lane));
  if (w_gate != nullptr) {
    const float gate = warp_sum(lane_dot(x, w_gate + ((size_t)e * ff + j) * width, width, lane));
    if (lane == 0) act[(size_t)p * ff + j] = from_f32<T>((activation == 0 ? gelu_erf(gate) : silu(gate)) * part);
    return;
  }
  if (lane == 0) {
    act[(size_t)p * ff + j] = from_f32<T>(activation == 0 ? gelu_erf(part) : silu(part));
  }
}

// out[t, i] = sum_k wts[t, k] * (W_down[e_k][i] . act[t * top + k]).  One warp per (token, i).
// w_down: [width, E, ff], the experts side by side in a row (the layout of one product over all experts).
template <typename T>
__global__ void moe_down_pairs_kernel(const T* __restrict__ act, const T* __restrict__ w_down, const int* __restrict__ idx,
                                      const float* __restrict__ wts, T* __restrict__ out, int n_tokens, int top, int width,
                                      int ff, int E) {
  pdl_wait();
  pdl_trigger();
  const int lane = threadIdx.x & 31;
  const long long id = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (id >= (long long)n_tokens * width) return;
  const int t = (int)(id / width), i = (int)(id - (long long)t * width);
  // a lane adds up its share of all chosen experts' rows, weighted; one sum over the warp at the end, so that the
  // rows of different experts are asked for together
  float total = 0.f;
#pragma unroll 4
  for (int k = 0; k < top; ++k) {
    const int e = idx[(size_t)t * top + k];
    const float part = lane_dot(act + ((size_t)t * top + k) * ff, w_down + ((size_t)i * E + e) * ff, ff, lane);
    total = fmaf(wts[(size_t)t * top + k], part, total);
  }
  total = warp_sum(total);
  if (lane == 0) out[(size_t)t * width + i] = from_f32<T>(total);
}

// `w_gate`: [E, ff, width] for gated experts, or null
AB_API int ab_moe_pairs_gated(const void* h, int dtype, int ld, const void* w_up, const void* w_gate, const void* w_down,
                              const int* idx, const float* wts, void* act, void* out, int n_tokens, int top, int width,
                              int ff, int E, int activation, cudaStream_t stream) {
  if (n_tokens <= 0) return AB_OK;
  if (top <= 0 || width <= 0 || ff <= 0 || E <= 0 || (activation != 0 && activation != 1)) return AB_BAD_ARG;
  const int wpb = 8;
  const long long up_warps = (long long)n_tokens * top * ff, down_warps = (long long)n_tokens * width;
  const long long up_blocks = (up_warps + wpb - 1) / wpb, down_blocks = (down_warps + wpb - 1) / wpb;
  if (up_blocks > 0x7fffffffLL || down_blocks > 0x7fffffffLL) return AB_BAD_ARG;
  if (dtype == AB_F32) {
    ab_launch(moe_up_pairs_kernel<float>, dim3((unsigned)up_blocks), dim3(wpb * 32), 0, stream, (const float*)h, ld,
              (const float*)w_up, (const float*)w_gate, idx, (float*)act, n_tokens * top, top, width, ff, activation);
    ab_launch(moe_down_pairs_kernel<float>, dim3((unsigned)down_blocks), dim3(wpb * 32), 0, stream, (const float*)act,
              (const float*)w_down, idx, wts, (float*)out, n_tokens, top, width, ff, E);
  } else if (dtype == AB_BF16) {
    ab_launch(moe_up_pairs_kernel<bf16>, dim3((unsigned)up_blocks), dim3(wpb * 32), 0, stream, (const bf16*)h, ld,
              (const bf16*)w_up, (const bf16*)w_gate, idx, (bf16*)act, n_tokens * top, top, width, ff, activation);
    ab_launch(moe_down_pairs_kernel<bf16>, dim3((unsigned)down_blocks), dim3(wpb * 32), 0, stream, (const bf16*)act,
              (const bf16*)w_down, idx, wts, (bf16*)out, n_tokens, top, width, ff, E);
  } else {
    return AB_BAD_ARG;
  }
  return ab_launch_status();
}

AB_API int ab_moe_pairs(const void* h, int dtype, int ld, const void* w_up, const void* w_down, const int* idx,
                        const float* wts, void* act, void* out, int n_tokens, int top, int width, int ff, int E,
                        int activation, cudaStream_t stream) {
  return ab_moe_pairs_gated(h, dtype, ld, w_up, nullptr, w_down, idx, wts, act, out, n_tokens, top, width, ff, E,
                            activation, stream);
}

// All experts at once, for steps of many tokens: up[t, e * ff + j] holds W_up[e][j] . h[t] for every expert
// (one product); in place it becomes act(up) * (the token's weight for expert e, 0 if e was not chosen), so
// that one product with the experts side by side, [width, E * ff], adds the chosen experts' outputs.
// Gated: a row of `up` holds the gates of all experts and then their up-projections (2 * E * ff numbers); the result
// takes the gates' place.
template <typename T>
__global__ void moe_weigh_all_kernel(T* __restrict__ up, const int* __restrict__ idx, const float* __restrict__ wts,
                                     int n_tokens, int top, int ff, int E, int activation, int gated) {
  const int t = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;       // column in [0, E * ff)
  if (c >= E * ff) return;
  const int e = c / ff;
  float g = 0.f;
  for (int k = 0; k < top; ++k)
    if (idx[(size_t)t * top + k] == e) g = wts[(size_t)t * top + k];
  T* x = up + (size_t)t * E * ff * (gated ? 2 : 1) + c;
  float y = 0.f;
  if (g != 0.f) {
    const float z = to_f32(*x);
    y = g * (activation == 0 ? gelu_erf(z) : silu(z));
    if (gated) y *= to_f32(x[(size_t)E * ff]);
  }
  *x = from_f32<T>(y);
}

// the same, eight bfloat16 columns per thread (ff a multiple of 8: the eight belong to one expert); the columns
// of experts that were not chosen are written without being read
__global__ void moe_weigh_all_bf16x8_kernel(bf16* __restrict__ up, const int* __restrict__ idx,
                                            const float* __restrict__ wts, int n_tokens, int top, int ff, int E,
                                            int activation, int gated) {
  const int t = blockIdx.y;
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (c >= E * ff) return;
  const int e = c / ff;
  float g = 0.f;
  for (int k = 0; k < top; ++k)
    if (idx[(size_t)t * top + k] == e) g = wts[(size_t)t * top + k];
  uint4* x = reinterpret_cast<uint4*>(up + (size_t)t * E * ff * (gated ? 2 : 1) + c);
  uint4 v = make_uint4(0, 0, 0, 0);
  if (g != 0.f) {
    v = *x;
    uint4 u = make_uint4(0, 0, 0, 0);
    if (gated) u = *reinterpret_cast<const uint4*>(up + (size_t)t * E * ff * 2 + (size_t)E * ff + c);
    __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&v);
    const __nv_bfloat162* pu = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 z = __bfloat1622float2(p[j]);
      z.x = g * (activation == 0 ? gelu_erf(z.x) : silu(z.x));
      z.y = g * (activation == 0 ? gelu_erf(z.y) : silu(z.y));
      if (gated) {
        const float2 m = __bfloat1622float2(pu[j]);
        z.x *= m.x;
        z.y *= m.y;
      }
      p[j] = __floats2bfloat162_rn(z.x, z.y);
    }
  }
  *x = v;
}

AB_API int ab_moe_weigh_all_gated(void* up, int dtype, const int* idx, const float* wts, int n_tokens, int top, int ff,
                                  int E, int activation, int gated, cudaStream_t stream) {
  if (n_tokens <= 0) return AB_OK;
  if (top <= 0 || ff <= 0 || E <= 0 || n_tokens > 65535 || (activation != 0 && activation != 1)) return AB_BAD_ARG;
  dim3 grid((unsigned)(((long long)E * ff + 255) / 256), (unsigned)n_tokens);
  if (dtype == AB_F32)
    moe_weigh_all_kernel<float><<<grid, 256, 0, stream>>>((float*)up, idx, wts, n_tokens, top, ff, E, activation, gated);
  else if (dtype == AB_BF16 && ff % 8 == 0 && (((uintptr_t)up) & 15) == 0) {
    dim3 grid8((unsigned)(((long long)E * ff / 8 + 255) / 256), (unsigned)n_tokens);
    moe_weigh_all_bf16x8_kernel<<<grid8, 256, 0, stream>>>((bf16*)up, idx, wts, n_tokens, top, ff, E, activation, gated);
  } else if (dtype == AB_BF16)
    moe_weigh_all_kernel<bf16><<<grid, 256, 0, stream>>>((bf16*)up, idx, wts, n_tokens, top, ff, E, activation, gated);
  else
    return AB_BAD_ARG;
  return ab_launch_status();
}

AB_API int ab_moe_weigh_all(void* up, int dtype, const int* idx, const float* wts, int n_tokens, int top, int ff, int E,
                            int activation, cudaStream_t stream) {
  return ab_moe_weigh_all_gated(up, dtype, idx, wts, n_tokens, top, ff, E, activation, 0, stream);
}
