// Linear attention with a fixed decay per head over packed sequences ("lightning attention").
//
// Per head, with q_t = silu(zq_t), k_t = silu(zk_t) (D dims), v_t = silu(zv_t) (V dims), a decay 0 < a <= 1 that
// the head keeps for good, and S_0 = 0:
//   S_t = a S_{t-1} + k_t v_t^T        [D, V]
//   o_t = S_t^T q_t
// The heads of a token are then divided by their common root mean square (all H*V values together), multiplied
// by a weight and by sigmoid(g_t).  The state, the decay and every sum are 32-bit.
//
// Two forms of the walk over the tokens share one entry point and give the same sums up to rounding:
//   walk     (steps of a few tokens per sequence) one CTA per (sequence, head, 32 columns of S): a column's D
//            entries are spread over the registers of 4 threads (4 warps, each holding a quarter of the rows for
//            32 columns); q and k of 8 tokens at a time are brought to shared memory with the activation
//            applied; a thread leaves its share of S^T q in shared memory, and the four shares are added in a
//            fixed order after the batch's last token;
//   stream   (prompts) a kernel first applies the activation to q | k | v in place; then one CTA per (sequence,
//            head, 8 or 32 columns) with a column spread over 16 or 4 threads, and the activated rows of 8 or 16
//            tokens at a time arriving in shared memory by cp.async, two buffers, so that the walk does not
//            wait for memory and one sequence spreads over many processors.  Few long sequences are cut into
//            pieces that are walked side by side: first every piece alone from a zero state (no outputs), which
//            leaves its own sum U_p; then S_p = a^len_p S_{p-1} + U_p along each sequence gives the state before
//            every piece; then every piece again from that state, with outputs.
// The state of a sequence is read when the step starts and written back when it ends, so a prompt may be cut
// anywhere and a decode step is the same code with one token.  The projections come as one float32 row per
// token: zq | zk | zv | g at given offsets.
//
// Options (retention: Sun et al., "Retentive Network: A Successor to Transformer for Large Language Models", has
// this recurrence with rotated q and k): no activation on q, k, v; a rotation by position of the first n_rot dims
// of every q and k vector (pairs (2i, 2i+1) or (i, i + n_rot/2), tables float32 [positions, n_rot/2]); k times a
// constant after the rotation; the root mean square taken per head instead of over all heads, with or without a
// weight; silu instead of sigmoid on the gate.
#include "common.cuh"
#include "launch.cuh"

struct LinAttnArgs {
  const float* proj;       // [T, ld]
  int ld, off_q, off_k, off_v, off_g;
  const float* decay;      // [H]
  float* state;            // [slots, H, D, V]
  int H, D, V;
  const int* cu_q;         // [B + 1]
  const int* slots;        // [B]
  const int* tok_seq;      // [T], -1: a row without a sequence
  float* o_raw;            // [T, H, V]
  int write_state;
  // the stream form on pieces of sequences (mode 1, 2); mode 0 walks whole sequences from state to state
  int mode;                // 1: a piece from zero, its sum to `pieces`, no outputs; 2: a piece from pieces[item], outputs
  const int* item_seq;     // [n_items] the sequence of each piece
  const int* item_t0;      // [n_items] its first packed token
  const int* item_t1;      // [n_items] one past its last
  float* pieces;           // [n_items, H, D, V]
  // what happens to the projections before the recurrence
  int act;                 // 1: silu on q, k, v; 0: none
  const float* cos_t;      // [positions, n_rot / 2] or null: no rotation
  const float* sin_t;
  int n_rot, pairing;      // pairing 0: (2i, 2i+1), 1: (i, i + n_rot/2)
  const int* tok_pos;      // [T]
  float k_scale;           // k is multiplied by this after the rotation
};

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }

// element d of a q or k vector `vec` (D floats as projected) after activation and rotation by position `pos`
__device__ __forceinline__ float la_prepared(const LinAttnArgs& a, const float* __restrict__ vec, int d, int pos) {
  float v = vec[d];
  if (a.act) v = silu_f(v);
  if (a.cos_t != nullptr && d < a.n_rot) {
    const int half = a.n_rot >> 1;
    int i, partner;
    bool first;
    if (a.pairing == 0) { i = d >> 1; first = (d & 1) == 0; partner = d ^ 1; }
    else { first = d < half; i = first ? d : d - half; partner = first ? d + half : d - half; }
    float p = vec[partner];
    if (a.act) p = silu_f(p);
    const float c = a.cos_t[(size_t)pos * half + i], sn = a.sin_t[(size_t)pos * half + i];
    v = first ? v * c - p * sn : v * c + p * sn;
  }
  return v;
}

#define LA_COLS 32
#define LA_SLICES 4
#define LA_TB 8

// DPT: rows of S per thread (a multiple of 4); the four slices cover 4 * DPT >= D rows
template <int DPT>
__global__ void __launch_bounds__(LA_COLS * LA_SLICES)
linattn_walk_kernel(LinAttnArgs a) {
  constexpr int DP = DPT * LA_SLICES;
  __shared__ __align__(16) float qs[LA_TB][DP];
  __shared__ __align__(16) float ks[LA_TB][DP];
  __shared__ float vs[LA_TB][LA_COLS];
  __shared__ float part[LA_TB][LA_SLICES][LA_COLS];
  pdl_wait();
  pdl_trigger();
  const int b = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * LA_COLS;
  const int t0 = a.cu_q[b], t1 = a.cu_q[b + 1];
  const int slot = a.slots[b];
  if (slot < 0 || t1 <= t0 || a.tok_seq[t0] < 0) return;
  const int tid = threadIdx.x, c = tid & 31, r = tid >> 5;
  const int D = a.D, V = a.V, col = c0 + c;
  const float lam = a.decay[h];
  float* st = a.state + ((size_t)slot * a.H + h) * (size_t)D * V;
  float s[DPT];
#pragma unroll
  for (int i = 0; i < DPT; ++i) {
    const int d = r * DPT + i;
    s[i] = (d < D && col < V) ? st[(size_t)d * V + col] : 0.f;
  }
  for (int tb = t0; tb < t1; tb += LA_TB) {
    const int n = min(LA_TB, t1 - tb);
    for (int i = tid; i < n * DP; i += LA_COLS * LA_SLICES) {
      const int tok = i / DP, d = i - tok * DP;
      const float* row = a.proj + (size_t)(tb + tok) * a.ld;
      const int pos = a.cos_t != nullptr ? a.tok_pos[tb + tok] : 0;
      qs[tok][d] = d < D ? la_prepared(a, row + a.off_q + h * D, d, pos) : 0.f;
      ks[tok][d] = d < D ? la_prepared(a, row + a.off_k + h * D, d, pos) * a.k_scale : 0.f;
    }
    for (int i = tid; i < n * LA_COLS; i += LA_COLS * LA_SLICES) {
      const int tok = i / LA_COLS, cc = i - tok * LA_COLS;
      float v = 0.f;
      if (c0 + cc < V) {
        v = a.proj[(size_t)(tb + tok) * a.ld + a.off_v + h * V + c0 + cc];
        if (a.act) v = silu_f(v);
      }
      vs[tok][cc] = v;
    }
    __syncthreads();
    for (int tok = 0; tok < n; ++tok) {
      const float vv = vs[tok][c];
      float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
      for (int i = 0; i < DPT; i += 4) {
        const float4 k4 = *reinterpret_cast<const float4*>(&ks[tok][r * DPT + i]);
        const float4 q4 = *reinterpret_cast<const float4*>(&qs[tok][r * DPT + i]);
        s[i] = fmaf(lam, s[i], k4.x * vv);
        acc0 = fmaf(s[i], q4.x, acc0);
        s[i + 1] = fmaf(lam, s[i + 1], k4.y * vv);
        acc1 = fmaf(s[i + 1], q4.y, acc1);
        s[i + 2] = fmaf(lam, s[i + 2], k4.z * vv);
        acc0 = fmaf(s[i + 2], q4.z, acc0);
        s[i + 3] = fmaf(lam, s[i + 3], k4.w * vv);
        acc1 = fmaf(s[i + 3], q4.w, acc1);
      }
      part[tok][r][c] = acc0 + acc1;
    }
    __syncthreads();
    for (int i = tid; i < n * LA_COLS; i += LA_COLS * LA_SLICES) {
      const int tok = i / LA_COLS, cc = i - tok * LA_COLS;
      if (c0 + cc < V)
        a.o_raw[((size_t)(tb + tok) * a.H + h) * V + c0 + cc] =
            ((part[tok][0][cc] + part[tok][1][cc]) + part[tok][2][cc]) + part[tok][3][cc];
    }
    __syncthreads();
  }
  if (a.write_state && col < V) {
#pragma unroll
    for (int i = 0; i < DPT; ++i) {
      const int d = r * DPT + i;
      if (d < D) st[(size_t)d * V + col] = s[i];
    }
  }
}

// silu in place on the columns [c0, c1) of every row that has a sequence
__global__ void linattn_activate_kernel(float* __restrict__ proj, int ld, int c0, int c1, const int* __restrict__ tok_seq,
                                        int n_tokens) {
  pdl_wait();
  pdl_trigger();
  const int w = c1 - c0;
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)n_tokens * w) return;
  const size_t t = i / w;
  if (tok_seq[t] < 0) return;
  float* p = proj + t * ld + c0 + (i - t * w);
  *p = silu_f(*p);
}

// q and k of every token in place: activation, rotation, k's constant.  One warp per (token, q or k vector).
__global__ void __launch_bounds__(128)
linattn_prepare_kernel(LinAttnArgs a, int n_tokens) {
  __shared__ float stage[4][256];
  pdl_wait();
  pdl_trigger();
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  const long long w = (long long)blockIdx.x * 4 + wib;
  if (w >= (long long)n_tokens * 2 * a.H) return;
  const int t = (int)(w / (2 * a.H)), vec = (int)(w - (long long)t * 2 * a.H);
  if (a.tok_seq[t] < 0) return;
  const bool is_k = vec >= a.H;
  const int h = is_k ? vec - a.H : vec;
  float* row = const_cast<float*>(a.proj) + (size_t)t * a.ld + (is_k ? a.off_k : a.off_q) + h * a.D;
  const int pos = a.cos_t != nullptr ? a.tok_pos[t] : 0;
  const float mul = is_k ? a.k_scale : 1.0f;
  float* x = stage[wib];
  for (int d = lane; d < a.D; d += 32) x[d] = la_prepared(a, row, d, pos) * mul;
  __syncwarp();
  for (int d = lane; d < a.D; d += 32) row[d] = x[d];
}

__device__ __forceinline__ void la_cp_async_16(void* smem, const void* gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem));
}
__device__ __forceinline__ void la_cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void la_cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

// The walk over activated rows.  DPT rows of S per thread, SL threads per column, 128 / SL columns per CTA, TB tokens
// per buffer.  Needs D, the offsets and ld to be multiples of 4 (16-byte pieces).
template <int DPT, int SL, int TB>
__global__ void __launch_bounds__(128)
linattn_stream_kernel(LinAttnArgs a) {
  constexpr int COLS = 128 / SL, DP = DPT * SL;
  extern __shared__ __align__(16) float la_smem[];
  float* qs = la_smem;                        // [2][TB][DP]
  float* ks = qs + 2 * TB * DP;               // [2][TB][DP]
  float* vs = ks + 2 * TB * DP;               // [2][TB][COLS]
  float* part = vs + 2 * TB * COLS;           // [TB][SL][COLS]
  pdl_wait();
  pdl_trigger();
  const int h = blockIdx.y, c0 = blockIdx.z * COLS;
  const int b = a.mode == 0 ? (int)blockIdx.x : a.item_seq[blockIdx.x];
  const int t0 = a.mode == 0 ? a.cu_q[b] : a.item_t0[blockIdx.x];
  const int t1 = a.mode == 0 ? a.cu_q[b + 1] : a.item_t1[blockIdx.x];
  const int slot = a.slots[b];
  if (slot < 0 || t1 <= t0 || a.tok_seq[t0] < 0) return;
  const int tid = threadIdx.x, c = tid % COLS, r = tid / COLS;
  const int D = a.D, V = a.V, col = c0 + c;
  const float lam = a.decay[h];
  const bool outputs = a.mode != 1;
  float* st = a.mode == 0 ? a.state + ((size_t)slot * a.H + h) * (size_t)D * V
                          : a.pieces + ((size_t)blockIdx.x * a.H + h) * (size_t)D * V;
  float s[DPT];
#pragma unroll
  for (int i = 0; i < DPT; ++i) {
    const int d = r * DPT + i;
    s[i] = (a.mode != 1 && d < D && col < V) ? st[(size_t)d * V + col] : 0.f;
  }
  // rows of S past D meet zeros: the padding of both buffers is cleared once and never written again
  for (int i = tid; i < 2 * TB * DP; i += 128) { qs[i] = 0.f; ks[i] = 0.f; }
  for (int i = tid; i < 2 * TB * COLS; i += 128) vs[i] = 0.f;
  __syncthreads();
  const int d4 = D >> 2;
  auto issue = [&](int tb, int stage) {
    const int n = min(TB, t1 - tb);
    for (int i = tid; i < n * d4; i += 128) {
      const int tok = i / d4, piece = i - tok * d4;
      const float* row = a.proj + (size_t)(tb + tok) * a.ld + h * D + piece * 4;
      if (outputs) la_cp_async_16(qs + (stage * TB + tok) * DP + piece * 4, row + a.off_q);
      la_cp_async_16(ks + (stage * TB + tok) * DP + piece * 4, row + a.off_k);
    }
    for (int i = tid; i < n * COLS; i += 128) {
      const int tok = i / COLS, cc = i - tok * COLS;
      if (c0 + cc < V) vs[(stage * TB + tok) * COLS + cc] = a.proj[(size_t)(tb + tok) * a.ld + a.off_v + h * V + c0 + cc];
    }
    la_cp_async_commit();
  };
  issue(t0, 0);
  int stage = 0;
  for (int tb = t0; tb < t1; tb += TB, stage ^= 1) {
    const int n = min(TB, t1 - tb);
    if (tb + TB < t1) { issue(tb + TB, stage ^ 1); la_cp_async_wait<1>(); } else { la_cp_async_wait<0>(); }
    __syncthreads();
    const float* qb = qs + stage * TB * DP + r * DPT;
    const float* kb = ks + stage * TB * DP + r * DPT;
    if (!outputs) {
      for (int tok = 0; tok < n; ++tok) {
        const float vv = vs[(stage * TB + tok) * COLS + c];
#pragma unroll
        for (int i = 0; i < DPT; i += 4) {
          const float4 k4 = *reinterpret_cast<const float4*>(kb + tok * DP + i);
          s[i] = fmaf(lam, s[i], k4.x * vv);
          s[i + 1] = fmaf(lam, s[i + 1], k4.y * vv);
          s[i + 2] = fmaf(lam, s[i + 2], k4.z * vv);
          s[i + 3] = fmaf(lam, s[i + 3], k4.w * vv);
        }
      }
      __syncthreads();
      continue;
    }
    for (int tok = 0; tok < n; ++tok) {
      const float vv = vs[(stage * TB + tok) * COLS + c];
      float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
      for (int i = 0; i < DPT; i += 4) {
        const float4 k4 = *reinterpret_cast<const float4*>(kb + tok * DP + i);
        const float4 q4 = *reinterpret_cast<const float4*>(qb + tok * DP + i);
        s[i] = fmaf(lam, s[i], k4.x * vv);
        acc0 = fmaf(s[i], q4.x, acc0);
        s[i + 1] = fmaf(lam, s[i + 1], k4.y * vv);
        acc1 = fmaf(s[i + 1], q4.y, acc1);
        s[i + 2] = fmaf(lam, s[i + 2], k4.z * vv);
        acc0 = fmaf(s[i + 2], q4.z, acc0);
        s[i + 3] = fmaf(lam, s[i + 3], k4.w * vv);
        acc1 = fmaf(s[i + 3], q4.w, acc1);
      }
      part[(tok * SL + r) * COLS + c] = acc0 + acc1;
    }
    __syncthreads();
    for (int i = tid; i < n * COLS; i += 128) {
      const int tok = i / COLS, cc = i - tok * COLS;
      if (c0 + cc < V) {
        float sum = 0.f;
#pragma unroll
        for (int j = 0; j < SL; ++j) sum += part[(tok * SL + j) * COLS + cc];
        a.o_raw[((size_t)(tb + tok) * a.H + h) * V + c0 + cc] = sum;
      }
    }
    // the next batch's first barrier comes before `part` and this stage's buffers are written again
  }
  if ((a.mode == 0 ? a.write_state : (a.mode == 1)) && col < V) {
#pragma unroll
    for (int i = 0; i < DPT; ++i) {
      const int d = r * DPT + i;
      if (d < D) st[(size_t)d * V + col] = s[i];
    }
  }
}

// Along each sequence: pieces[p] <- the state before piece p, and the state moves on by a^len_p S + U_p; at the
// end it is the sequence's new state.  A thread per element of S.
__global__ void linattn_combine_kernel(LinAttnArgs a, const int* __restrict__ seq_first, const int* __restrict__ seq_count,
                                       int n_seqs) {
  pdl_wait();
  pdl_trigger();
  const size_t per_head = (size_t)a.D * a.V, per_seq = per_head * a.H;
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= per_seq * n_seqs) return;
  const int b = (int)(i / per_seq);
  const size_t e = i - (size_t)b * per_seq;
  const int h = (int)(e / per_head);
  const int slot = a.slots[b], n = seq_count[b], first = seq_first[b];
  if (slot < 0 || n <= 0 || a.tok_seq[a.item_t0[first]] < 0) return;
  const float lam = a.decay[h];
  float* st = a.state + (size_t)slot * per_seq + e;
  float S = *st;
  int len_known = -1;
  float pw = 1.f;
  for (int p = first; p < first + n; ++p) {
    const int len = a.item_t1[p] - a.item_t0[p];
    // a^len as 2^(len log2 a): where the power is not negligible its relative error stays below 2e-6 (the
    // library's powf costs a hundred instructions, which for every element of S was most of this kernel)
    if (len != len_known) { pw = lam >= 1.f ? 1.f : exp2f((float)len * log2f(lam)); len_known = len; }
    float* u = a.pieces + (size_t)p * per_seq + e;
    const float U = *u;
    *u = S;
    S = fmaf(pw, S, U);
  }
  if (a.write_state) *st = S;
}

// The same, four elements per thread (D * V a multiple of 4) and the pieces' sums of four pieces fetched before any of
// them is overwritten, so that a thread's loads do not wait for one another.
__global__ void linattn_combine4_kernel(LinAttnArgs a, const int* __restrict__ seq_first, const int* __restrict__ seq_count,
                                        int n_seqs) {
  pdl_wait();
  pdl_trigger();
  const unsigned per_head4 = (unsigned)(a.D * a.V) >> 2, per_seq4 = per_head4 * a.H;
  const unsigned i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= per_seq4 * (unsigned)n_seqs) return;
  const int b = (int)(i / per_seq4);
  const unsigned e = i - (unsigned)b * per_seq4;
  const int h = (int)(e / per_head4);
  const int slot = a.slots[b], n = seq_count[b], first = seq_first[b];
  if (slot < 0 || n <= 0 || a.tok_seq[a.item_t0[first]] < 0) return;
  const float lam = a.decay[h], l2 = lam >= 1.f ? 0.f : log2f(lam);
  float4* st = reinterpret_cast<float4*>(a.state) + (size_t)slot * per_seq4 + e;
  float4* pieces = reinterpret_cast<float4*>(a.pieces) + e;
  float4 S = *st;
  for (int p0 = first; p0 < first + n; p0 += 4) {
    const int m = min(4, first + n - p0);
    float4 U[4];
    float pw[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (j < m) {
        U[j] = pieces[(size_t)(p0 + j) * per_seq4];
        pw[j] = exp2f((float)(a.item_t1[p0 + j] - a.item_t0[p0 + j]) * l2);
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (j < m) {
        pieces[(size_t)(p0 + j) * per_seq4] = S;
        S.x = fmaf(pw[j], S.x, U[j].x);
        S.y = fmaf(pw[j], S.y, U[j].y);
        S.z = fmaf(pw[j], S.z, U[j].z);
        S.w = fmaf(pw[j], S.w, U[j].w);
      }
    }
  }
  if (a.write_state) *st = S;
}

template <int DPT, int SL, int TB>
static int launch_stream(const LinAttnArgs& a, int n_seqs, cudaStream_t stream) {
  constexpr int COLS = 128 / SL, DP = DPT * SL;
  const size_t smem = (size_t)(4 * TB * DP + 2 * TB * COLS + TB * SL * COLS) * sizeof(float);
  const unsigned col_tiles = (unsigned)((a.V + COLS - 1) / COLS);
  if (col_tiles > 65535) return AB_BAD_ARG;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(linattn_stream_kernel<DPT, SL, TB>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) return AB_CUDA_ERR + (int)e;
  }
  ab_launch(linattn_stream_kernel<DPT, SL, TB>, dim3((unsigned)n_seqs, (unsigned)a.H, col_tiles), dim3(128), smem, stream, a);
  return ab_launch_status();
}

// the stream kernel's form for D; `rows`: sequences (mode 0) or pieces
static int stream_dispatch(const LinAttnArgs& a, int rows, cudaStream_t stream) {
  const int D = a.D;
  if (D % 64 == 0 && D <= 64) return launch_stream<4, 16, 16>(a, rows, stream);
  if (D % 64 == 0 && D <= 128) return launch_stream<8, 16, 16>(a, rows, stream);
  if (D % 64 == 0) return launch_stream<16, 16, 8>(a, rows, stream);
  if (D <= 16) return launch_stream<4, 4, 16>(a, rows, stream);
  if (D <= 32) return launch_stream<8, 4, 16>(a, rows, stream);
  if (D <= 64) return launch_stream<16, 4, 16>(a, rows, stream);
  if (D <= 128) return launch_stream<32, 4, 16>(a, rows, stream);
  return launch_stream<64, 4, 8>(a, rows, stream);
}

// columns of S per CTA of the stream form (its callers plan their pieces by the number of CTAs)
AB_API int ab_linear_attention_stream_cols(int D) { return D % 64 == 0 ? 8 : 32; }

// out[t, j] = o[t, j] / rms(o[t, :]) * weight[j] * sigmoid(g[t, j]) over all H*V values of a token; a block per token
template <typename T>
__global__ void linattn_output_kernel(const float* __restrict__ o_raw, const float* __restrict__ proj, int ld, int off_g,
                                      const float* __restrict__ weight, const int* __restrict__ tok_seq,
                                      T* __restrict__ out, int n, float eps, int gate_silu) {
  __shared__ float scratch[32];
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  T* y = out + (size_t)t * n;
  if (tok_seq[t] < 0) {
    for (int j = threadIdx.x; j < n; j += blockDim.x) y[j] = from_f32<T>(0.f);
    return;
  }
  const float* o = o_raw + (size_t)t * n;
  float ss = 0.f;
  for (int j = threadIdx.x; j < n; j += blockDim.x) ss += o[j] * o[j];
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)n + eps);
  const float* g = proj + (size_t)t * ld + off_g;
  for (int j = threadIdx.x; j < n; j += blockDim.x) {
    const float gate = (gate_silu ? g[j] : 1.0f) / (1.0f + expf(-g[j]));
    y[j] = from_f32<T>(o[j] * inv * weight[j] * gate);
  }
}

// The root mean square per head: out[t, h, j] = o[t, h, j] / rms(o[t, h, :]) * weight[h, j] (weight null: 1) * gate.
// One warp per (token, head).
template <typename T>
__global__ void __launch_bounds__(128)
linattn_output_head_kernel(const float* __restrict__ o_raw, const float* __restrict__ proj, int ld, int off_g,
                           const float* __restrict__ weight, const int* __restrict__ tok_seq, T* __restrict__ out,
                           int n_tokens, int H, int V, float eps, int gate_silu) {
  pdl_wait();
  pdl_trigger();
  const int lane = threadIdx.x & 31;
  const long long w = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (w >= (long long)n_tokens * H) return;
  const int t = (int)(w / H), h = (int)(w - (long long)t * H);
  T* y = out + (size_t)w * V;
  if (tok_seq[t] < 0) {
    for (int j = lane; j < V; j += 32) y[j] = from_f32<T>(0.f);
    return;
  }
  const float* o = o_raw + (size_t)w * V;
  float ss = 0.f;
  for (int j = lane; j < V; j += 32) ss += o[j] * o[j];
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / (float)V + eps);
  const float* g = proj + (size_t)t * ld + off_g + h * V;
  for (int j = lane; j < V; j += 32) {
    const float gate = (gate_silu ? g[j] : 1.0f) / (1.0f + expf(-g[j]));
    y[j] = from_f32<T>(o[j] * inv * (weight != nullptr ? weight[h * V + j] : 1.0f) * gate);
  }
}

// The same with the token's values in registers (one pass over memory, 16-byte accesses): 256 threads, NV pieces of
// four per thread; n, ld and off_g multiples of 4, n up to 1024 * NV.
template <typename T, int NV>
__global__ void __launch_bounds__(256)
linattn_output_vec_kernel(const float* __restrict__ o_raw, const float* __restrict__ proj, int ld, int off_g,
                          const float* __restrict__ weight, const int* __restrict__ tok_seq, T* __restrict__ out, int n,
                          float eps, int gate_silu) {
  __shared__ float scratch[32];
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x, n4 = n >> 2;
  T* y = out + (size_t)t * n;
  if (tok_seq[t] < 0) {
    for (int j = threadIdx.x; j < n; j += blockDim.x) y[j] = from_f32<T>(0.f);
    return;
  }
  const float4* o = reinterpret_cast<const float4*>(o_raw + (size_t)t * n);
  const float4* g = reinterpret_cast<const float4*>(proj + (size_t)t * ld + off_g);
  const float4* wr = reinterpret_cast<const float4*>(weight);
  float4 ov[NV], gv[NV];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int i = threadIdx.x + k * 256;
    if (i < n4) {
      ov[k] = o[i];
      gv[k] = g[i];
      ss += (ov[k].x * ov[k].x + ov[k].y * ov[k].y) + (ov[k].z * ov[k].z + ov[k].w * ov[k].w);
    }
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)n + eps);
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int i = threadIdx.x + k * 256;
    if (i < n4) {
      const float4 wv = wr[i];
      y[4 * i] = from_f32<T>(ov[k].x * inv * wv.x * (gate_silu ? gv[k].x : 1.0f) / (1.0f + expf(-gv[k].x)));
      y[4 * i + 1] = from_f32<T>(ov[k].y * inv * wv.y * (gate_silu ? gv[k].y : 1.0f) / (1.0f + expf(-gv[k].y)));
      y[4 * i + 2] = from_f32<T>(ov[k].z * inv * wv.z * (gate_silu ? gv[k].z : 1.0f) / (1.0f + expf(-gv[k].z)));
      y[4 * i + 3] = from_f32<T>(ov[k].w * inv * wv.w * (gate_silu ? gv[k].w : 1.0f) / (1.0f + expf(-gv[k].w)));
    }
  }
}

// silu in place, four columns per thread (c0, c1 and ld multiples of 4)
__global__ void linattn_activate4_kernel(float* __restrict__ proj, int ld, int c0, int c1, const int* __restrict__ tok_seq,
                                         int n_tokens) {
  pdl_wait();
  pdl_trigger();
  const int w4 = (c1 - c0) >> 2;
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)n_tokens * w4) return;
  const size_t t = i / w4;
  if (tok_seq[t] < 0) return;
  float4* p = reinterpret_cast<float4*>(proj + t * ld + c0) + (i - t * w4);
  float4 v = *p;
  v.x = silu_f(v.x); v.y = silu_f(v.y); v.z = silu_f(v.z); v.w = silu_f(v.w);
  *p = v;
}

AB_API int ab_linear_attention_max_dim() { return 64 * LA_SLICES; }

// `stream_from`: steps with more than this many tokens per sequence on average take the `stream` form (it rewrites
// q | k | v of `proj` in place with their activations).  With n_items > 0 the stream form walks pieces of the
// sequences side by side: piece p is the packed tokens item_t0[p] .. item_t1[p] - 1 of sequence item_seq[p]; the pieces
// of sequence b are seq_first[b] .. seq_first[b] + seq_count[b] - 1, in order, and cover its tokens; `pieces` is
// scratch, float [n_items, H, D, V].
//
// The options: `act` 1 = silu on q, k, v, 0 = none; cos_t, sin_t (or null), n_rot, pairing, tok_pos: the rotation of q
// and k; k_scale; `head_norm` 1 = the root mean square per head, 0 = over all heads; `weight` may be null with
// head_norm (no weight); `gate_silu` 1 = silu(g), 0 = sigmoid(g).
AB_API int ab_linear_attention_step_opts(const float* proj, int ld, int off_q, int off_k, int off_v, int off_g,
                                         const float* decay, float* state, int H, int D, int V, const int* cu_q,
                                         const int* slots, const int* tok_seq, int n_seqs, int n_tokens, float* o_raw,
                                         const float* weight, float eps, void* out, int out_dtype, int write_state,
                                         int stream_from, const int* item_seq, const int* item_t0, const int* item_t1,
                                         int n_items, float* pieces, const int* seq_first, const int* seq_count,
                                         int act, const float* cos_t, const float* sin_t, int n_rot, int pairing,
                                         const int* tok_pos, float k_scale, int head_norm, int gate_silu,
                                         cudaStream_t stream) {
  if (n_seqs <= 0 || n_tokens <= 0) return AB_OK;
  if (H <= 0 || D <= 0 || V <= 0 || D > 64 * LA_SLICES || H > 65535) return AB_BAD_ARG;
  if (n_rot < 0 || n_rot > D || (n_rot & 1) || pairing < 0 || pairing > 1) return AB_BAD_ARG;
  if (!cos_t || !sin_t || n_rot == 0) { cos_t = sin_t = nullptr; n_rot = 0; }
  if (cos_t && !tok_pos) return AB_BAD_ARG;
  if (!weight && !head_norm) return AB_BAD_ARG;
  LinAttnArgs a{proj, ld, off_q, off_k, off_v, off_g, decay, state, H, D, V, cu_q, slots, tok_seq, o_raw, write_state,
                0, nullptr, nullptr, nullptr, nullptr, act ? 1 : 0, cos_t, sin_t, n_rot, pairing, tok_pos, k_scale};
  const bool plain_qk = cos_t == nullptr && k_scale == 1.0f;     // q and k need the activation at most
  const unsigned col_tiles = (unsigned)((V + LA_COLS - 1) / LA_COLS);
  if (col_tiles > 65535) return AB_BAD_ARG;
  int rc;
  const bool aligned = D % 4 == 0 && ld % 4 == 0 && off_q % 4 == 0 && off_k % 4 == 0;
  if (aligned && n_tokens > stream_from * n_seqs) {
    // prompts: activation (and rotation, and k's constant) in place, then the walk on rows that cp.async brings
    if (!(off_k == off_q + H * D && off_v == off_k + H * D)) return AB_BAD_ARG;   // q | k | v side by side
    if (!plain_qk) {
      const long long warps = (long long)n_tokens * 2 * H;
      ab_launch(linattn_prepare_kernel, dim3((unsigned)((warps + 3) / 4)), dim3(128), 0, stream, a, n_tokens);
      rc = ab_launch_status();
      if (rc) return rc;
    }
    // what is left for the activation: q | k | v, or v alone when q and k were prepared above
    const int c0 = plain_qk ? (off_q < off_k ? off_q : off_k) : off_v, c1 = off_v + H * V;
    if (act) {
      const size_t total = (size_t)n_tokens * (c1 - c0);
      if (c0 % 4 == 0 && (c1 - c0) % 4 == 0)
        ab_launch(linattn_activate4_kernel, dim3((unsigned)((total / 4 + 255) / 256)), dim3(256), 0, stream,
                  const_cast<float*>(proj), ld, c0, c1, tok_seq, n_tokens);
      else
        ab_launch(linattn_activate_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream,
                  const_cast<float*>(proj), ld, c0, c1, tok_seq, n_tokens);
      rc = ab_launch_status();
      if (rc) return rc;
    }
    if (n_items > 0) {
      if (!item_seq || !item_t0 || !item_t1 || !pieces || !seq_first || !seq_count) return AB_BAD_ARG;
      a.item_seq = item_seq; a.item_t0 = item_t0; a.item_t1 = item_t1; a.pieces = pieces;
      a.mode = 1;
      rc = stream_dispatch(a, n_items, stream);
      if (rc) return rc;
      const size_t elems = (size_t)n_seqs * H * D * V;
      if ((D * V) % 4 == 0 && elems / 4 < 0x7fffffffULL)
        ab_launch(linattn_combine4_kernel, dim3((unsigned)((elems / 4 + 255) / 256)), dim3(256), 0, stream, a, seq_first,
                  seq_count, n_seqs);
      else
        ab_launch(linattn_combine_kernel, dim3((unsigned)((elems + 255) / 256)), dim3(256), 0, stream, a, seq_first,
                  seq_count, n_seqs);
      rc = ab_launch_status();
      if (rc) return rc;
      a.mode = 2;
      rc = stream_dispatch(a, n_items, stream);
    } else {
      rc = stream_dispatch(a, n_seqs, stream);
    }
  } else {
    dim3 grid((unsigned)n_seqs, (unsigned)H, col_tiles), block(LA_COLS * LA_SLICES);
    const int dpt = (D + LA_SLICES - 1) / LA_SLICES;
    if (dpt <= 4) ab_launch(linattn_walk_kernel<4>, grid, block, 0, stream, a);
    else if (dpt <= 8) ab_launch(linattn_walk_kernel<8>, grid, block, 0, stream, a);
    else if (dpt <= 16) ab_launch(linattn_walk_kernel<16>, grid, block, 0, stream, a);
    else if (dpt <= 32) ab_launch(linattn_walk_kernel<32>, grid, block, 0, stream, a);
    else ab_launch(linattn_walk_kernel<64>, grid, block, 0, stream, a);
    rc = ab_launch_status();
  }
  if (rc) return rc;
  const int n = H * V;
  if (head_norm) {
    const long long warps = (long long)n_tokens * H;
    const unsigned blocks = (unsigned)((warps + 3) / 4);
    if (out_dtype == AB_F32)
      ab_launch(linattn_output_head_kernel<float>, dim3(blocks), dim3(128), 0, stream, (const float*)o_raw, proj, ld, off_g,
                weight, tok_seq, (float*)out, n_tokens, H, V, eps, gate_silu);
    else if (out_dtype == AB_BF16)
      ab_launch(linattn_output_head_kernel<bf16>, dim3(blocks), dim3(128), 0, stream, (const float*)o_raw, proj, ld, off_g,
                weight, tok_seq, (bf16*)out, n_tokens, H, V, eps, gate_silu);
    else
      return AB_BAD_ARG;
    return ab_launch_status();
  }
  if (n % 4 == 0 && n <= 8192 && ld % 4 == 0 && off_g % 4 == 0 && (out_dtype == AB_F32 || out_dtype == AB_BF16)) {
#define AB_GO(T, NV) ab_launch(linattn_output_vec_kernel<T, NV>, dim3((unsigned)n_tokens), dim3(256), 0, stream, \
                               (const float*)o_raw, proj, ld, off_g, weight, tok_seq, (T*)out, n, eps, gate_silu)
    if (out_dtype == AB_F32) {
      if (n <= 1024) AB_GO(float, 1); else if (n <= 2048) AB_GO(float, 2); else if (n <= 4096) AB_GO(float, 4); else AB_GO(float, 8);
    } else {
      if (n <= 1024) AB_GO(bf16, 1); else if (n <= 2048) AB_GO(bf16, 2); else if (n <= 4096) AB_GO(bf16, 4); else AB_GO(bf16, 8);
    }
#undef AB_GO
    return ab_launch_status();
  }
  const int threads = n >= 1024 ? 256 : 128;
  if (out_dtype == AB_F32)
    ab_launch(linattn_output_kernel<float>, dim3((unsigned)n_tokens), dim3(threads), 0, stream, (const float*)o_raw, proj,
              ld, off_g, weight, tok_seq, (float*)out, n, eps, gate_silu);
  else if (out_dtype == AB_BF16)
    ab_launch(linattn_output_kernel<bf16>, dim3((unsigned)n_tokens), dim3(threads), 0, stream, (const float*)o_raw, proj,
              ld, off_g, weight, tok_seq, (bf16*)out, n, eps, gate_silu);
  else
    return AB_BAD_ARG;
  return ab_launch_status();
}

// The form without options: silu on q, k, v, no rotation, the root mean square over all heads, sigmoid(g).
AB_API int ab_linear_attention_step(const float* proj, int ld, int off_q, int off_k, int off_v, int off_g,
                                    const float* decay, float* state, int H, int D, int V, const int* cu_q,
                                    const int* slots, const int* tok_seq, int n_seqs, int n_tokens, float* o_raw,
                                    const float* weight, float eps, void* out, int out_dtype, int write_state,
                                    int stream_from, const int* item_seq, const int* item_t0, const int* item_t1,
                                    int n_items, float* pieces, const int* seq_first, const int* seq_count,
                                    cudaStream_t stream) {
  return ab_linear_attention_step_opts(proj, ld, off_q, off_k, off_v, off_g, decay, state, H, D, V, cu_q, slots, tok_seq,
                                       n_seqs, n_tokens, o_raw, weight, eps, out, out_dtype, write_state, stream_from,
                                       item_seq, item_t0, item_t1, n_items, pieces, seq_first, seq_count, 1, nullptr,
                                       nullptr, 0, 0, nullptr, 1.0f, 0, 0, stream);
}
