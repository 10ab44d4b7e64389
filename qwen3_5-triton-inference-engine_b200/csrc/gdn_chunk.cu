// Gated-DeltaNet chunk-64 prefill as the reference's three operators, with its intermediate tensors:
//   b200_gdn_chunk_prepare_wy <-> triton_kernels/gdn_recurrent_prefill.py:703-784 (kernel :248-396)
//   b200_gdn_chunk_state      <-> triton_kernels/gdn_recurrent_prefill.py:825-909 (kernel :404-537)
//   b200_gdn_chunk_output     <-> triton_kernels/gdn_recurrent_prefill.py:935-1006 (kernel :563-690)
// Per chunk (G = cumsum(g) inside the chunk, S_in the state entering it):
//   L[t,i] = beta_t exp(G_t - G_i) <k_t,k_i> (i<t);  P = (I+L)^-1;  u = P (beta v);  w = P (beta exp(G) k)
//   delta = u - w S_in;  S_out = exp(G_last) S_in + sum_t k_t (exp(G_last - G_t) delta_t)^T
//   o_t = exp(G_t) q_t^T S_in + sum_{i<=t} <q_t,k_i> exp(G_t - G_i) delta_i
// All products are true fp32 FMAs here (the reference needs 3xTF32 to hold its 5e-4 state tolerance; plain fp32
// is at least as accurate).  These kernels keep the reference's data flow through HBM so that each operator can be
// swapped individually.
#include "b200_attn.h"
#include "common.cuh"

namespace b200 {

constexpr int GC_THREADS = 256;
constexpr int GC_PITCH = GDN_D + 4;   // fp32 row pitch of [64][128] tiles (16-byte aligned rows, banks shifted by 4)
constexpr int GC_LP = CHUNK + 1;      // pitch of [64][64] tiles

// Where a CTA's chunk lives.  Single sequence (cu_seqlens == nullptr): chunk = blockIdx.x of `token_num` tokens.
// Packed batch: blockIdx.z = sequence, blockIdx.x = chunk inside it; chunks of all sequences are numbered
// consecutively (sequence after sequence), which is also how the intermediates are laid out.
struct ChunkPos {
  int chunk;      // global chunk index (row of the intermediates)
  int t0;         // first token of the chunk in the packed buffer
  int t_end;      // one past the last token of the sequence
  bool valid;
};
__device__ __forceinline__ ChunkPos locate_chunk(const int32_t* cu_seqlens, int token_num) {
  ChunkPos c;
  if (cu_seqlens == nullptr) {
    c.chunk = blockIdx.x;
    c.t0 = blockIdx.x * CHUNK;
    c.t_end = token_num;
    c.valid = true;
    return c;
  }
  const int b = blockIdx.z;
  const int start = cu_seqlens[b], len = cu_seqlens[b + 1] - start;
  int base = 0;
  for (int i = 0; i < b; ++i) base += (cu_seqlens[i + 1] - cu_seqlens[i] + CHUNK - 1) / CHUNK;
  c.chunk = base + blockIdx.x;
  c.t0 = start + blockIdx.x * CHUNK;
  c.t_end = start + len;
  c.valid = blockIdx.x * CHUNK < len;
  return c;
}

// ---------------------------------------------------------------------------------------------------- prepare_wy
constexpr int PW_SMEM = (2 * CHUNK * GC_PITCH + 2 * CHUNK * GC_LP + 4 * CHUNK) * 4;

__global__ void __launch_bounds__(GC_THREADS)
gdn_chunk_prepare_wy_kernel(const __nv_bfloat16* __restrict__ k, int64_t k_t, int64_t k_h,
                            const __nv_bfloat16* __restrict__ v, int64_t v_t, int64_t v_h,
                            const float* __restrict__ beta, int64_t be_t, int64_t be_h, const float* __restrict__ g,
                            int64_t g_t, int64_t g_h, float* __restrict__ w, float* __restrict__ u_base,
                            float* __restrict__ g_cumsum, int token_num, int heads,
                            const int32_t* __restrict__ cu_seqlens) {
  extern __shared__ __align__(16) float sm[];
  const ChunkPos pos = locate_chunk(cu_seqlens, token_num);
  if (!pos.valid) return;
  token_num = pos.t_end;
  float* kf = sm;                            // [64][GC_PITCH]
  float* vf = kf + CHUNK * GC_PITCH;         // [64][GC_PITCH]
  float* lower = vf + CHUNK * GC_PITCH;      // [64][GC_LP]
  float* inv = lower + CHUNK * GC_LP;        // [64][GC_LP]
  float* gs = inv + CHUNK * GC_LP;           // g, then G
  float* bs = gs + CHUNK;                    // beta
  float* es = bs + CHUNK;                    // exp(G)
  const int chunk = pos.chunk, h = blockIdx.y, tid = threadIdx.x;
  const int t0 = pos.t0;

  for (int i = tid; i < CHUNK * GDN_D; i += GC_THREADS) {
    const int r = i / GDN_D, c = i % GDN_D;
    const int64_t t = t0 + r;
    const bool ok = t < token_num;
    kf[r * GC_PITCH + c] = ok ? __bfloat162float(k[t * k_t + h * k_h + c]) : 0.f;
    vf[r * GC_PITCH + c] = ok ? __bfloat162float(v[t * v_t + h * v_h + c]) : 0.f;
  }
  if (tid < CHUNK) {
    const int64_t t = t0 + tid;
    const bool ok = t < token_num;
    gs[tid] = ok ? g[t * g_t + h * g_h] : 0.f;
    bs[tid] = ok ? beta[t * be_t + h * be_h] : 0.f;
  }
  __syncthreads();
  if (tid == 0) {
    float run = 0.f;
    for (int i = 0; i < CHUNK; ++i) {
      run += gs[i];
      gs[i] = run;
    }
  }
  __syncthreads();
  if (tid < CHUNK) {
    g_cumsum[(static_cast<int64_t>(chunk) * heads + h) * CHUNK + tid] = gs[tid];
    es[tid] = expf(gs[tid]);
  }
  // ---- lower[t][i] = beta_t exp(G_t - G_i) <k_t, k_i> for i < t, both tokens valid
  {
    const int t = tid >> 2, ig = (tid & 3) * 16;
    const float4* kt = reinterpret_cast<const float4*>(kf + t * GC_PITCH);
    for (int ii = 0; ii < 16; ++ii) {
      const int i = ig + ii;
      float val = 0.f;
      if (i < t && t0 + t < token_num) {
        const float4* ki = reinterpret_cast<const float4*>(kf + i * GC_PITCH);
        float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll 8
        for (int d = 0; d < GDN_D / 4; ++d) {
          const float4 x = kt[d], y = ki[d];
          a0 = fmaf(x.x, y.x, a0);
          a1 = fmaf(x.y, y.y, a1);
          a2 = fmaf(x.z, y.z, a2);
          a3 = fmaf(x.w, y.w, a3);
        }
        val = bs[t] * expf(gs[t] - gs[i]) * ((a0 + a1) + (a2 + a3));
      }
      lower[t * GC_LP + i] = val;
    }
  }
  __syncthreads();
  // ---- inv = (I + lower)^-1 by forward substitution; thread j owns column j (columns are independent)
  if (tid < CHUNK) {
    const int j = tid;
    for (int row = 0; row < CHUNK; ++row) {
      float val;
      if (row < j) val = 0.f;
      else if (row == j) val = 1.f;
      else {
        float a0 = 0.f, a1 = 0.f;
        int i = j;
        for (; i + 1 < row; i += 2) {
          a0 = fmaf(lower[row * GC_LP + i], inv[i * GC_LP + j], a0);
          a1 = fmaf(lower[row * GC_LP + i + 1], inv[(i + 1) * GC_LP + j], a1);
        }
        if (i < row) a0 = fmaf(lower[row * GC_LP + i], inv[i * GC_LP + j], a0);
        val = -(a0 + a1);
      }
      inv[row * GC_LP + j] = val;
    }
  }
  // ---- right-hand sides in place: vf <- beta v, kf <- beta exp(G) k
  __syncthreads();
  for (int i = tid; i < CHUNK * GDN_D; i += GC_THREADS) {
    const int r = i / GDN_D, c = i % GDN_D;
    vf[r * GC_PITCH + c] *= bs[r];
    kf[r * GC_PITCH + c] *= bs[r] * es[r];
  }
  __syncthreads();
  // ---- u = inv @ vf, w = inv @ kf : warp = 8 rows, lane = 4 columns
  {
    const int r0 = (tid >> 5) * 8, c0 = (tid & 31) * 4;
    const int64_t out_base = (static_cast<int64_t>(chunk) * heads + h) * CHUNK * GDN_D;
#pragma unroll
    for (int which = 0; which < 2; ++which) {
      const float* rhs = which == 0 ? vf : kf;
      float acc[8][4];
#pragma unroll
      for (int r = 0; r < 8; ++r) acc[r][0] = acc[r][1] = acc[r][2] = acc[r][3] = 0.f;
      for (int i = 0; i < r0 + 8; ++i) {  // inv is lower triangular: columns past the last row of the group are zero
        const float4 b = *reinterpret_cast<const float4*>(rhs + i * GC_PITCH + c0);
#pragma unroll
        for (int r = 0; r < 8; ++r) {
          const float a = inv[(r0 + r) * GC_LP + i];
          acc[r][0] = fmaf(a, b.x, acc[r][0]);
          acc[r][1] = fmaf(a, b.y, acc[r][1]);
          acc[r][2] = fmaf(a, b.z, acc[r][2]);
          acc[r][3] = fmaf(a, b.w, acc[r][3]);
        }
      }
      float* dst = (which == 0 ? u_base : w) + out_base;
#pragma unroll
      for (int r = 0; r < 8; ++r)
        *reinterpret_cast<float4*>(dst + (r0 + r) * GDN_D + c0) = make_float4(acc[r][0], acc[r][1], acc[r][2], acc[r][3]);
    }
  }
}

// ---------------------------------------------------------------------------------------------------- chunk_state
constexpr int CS_BV = 16;  // value columns per CTA
constexpr int CS_SMEM = (2 * CHUNK * GC_PITCH + GDN_D * CS_BV + 2 * CHUNK * CS_BV + 2 * CHUNK) * 4;

__global__ void __launch_bounds__(GC_THREADS)
gdn_chunk_state_kernel(const __nv_bfloat16* __restrict__ k, int64_t k_t, int64_t k_h, const float* __restrict__ w,
                       const float* __restrict__ u_base, const float* __restrict__ g_cumsum, float* __restrict__ delta,
                       float* __restrict__ chunk_state, float* __restrict__ final_state, int token_num, int num_chunks,
                       int heads, const int32_t* __restrict__ cu_seqlens) {
  extern __shared__ __align__(16) float sm[];
  // packed batch: blockIdx.z = sequence; its chunks are [chunk_base, chunk_base + num_chunks)
  int chunk_base = 0, tok_base = 0;
  if (cu_seqlens != nullptr) {
    const int b = blockIdx.z;
    for (int i = 0; i < b; ++i) chunk_base += (cu_seqlens[i + 1] - cu_seqlens[i] + CHUNK - 1) / CHUNK;
    tok_base = cu_seqlens[b];
    token_num = cu_seqlens[b + 1] - tok_base;
    num_chunks = (token_num + CHUNK - 1) / CHUNK;
  }
  float* wf = sm;                           // [64][GC_PITCH]
  float* kf = wf + CHUNK * GC_PITCH;        // [64][GC_PITCH]
  float* st = kf + CHUNK * GC_PITCH;        // [128][16]
  float* dl = st + GDN_D * CS_BV;           // delta [64][16]
  float* de = dl + CHUNK * CS_BV;           // delta * exp(G_last - G) [64][16]
  float* gs = de + CHUNK * CS_BV;           // G [64]
  float* dec = gs + CHUNK;                  // exp(G_last - G) (0 for padded tokens)
  const int h = blockIdx.x, v0 = blockIdx.y * CS_BV, tid = threadIdx.x;

  for (int i = tid; i < GDN_D * CS_BV; i += GC_THREADS) st[i] = 0.f;
  __syncthreads();
  for (int c = 0; c < num_chunks; ++c) {
    const int64_t ch = static_cast<int64_t>(chunk_base + c) * heads + h;
    // state entering the chunk
    for (int i = tid; i < GDN_D * CS_BV / 4; i += GC_THREADS) {
      const int kk = i / (CS_BV / 4), q4 = i % (CS_BV / 4);
      *reinterpret_cast<float4*>(chunk_state + (ch * GDN_D + kk) * GDN_D + v0 + q4 * 4) =
          *reinterpret_cast<const float4*>(st + kk * CS_BV + q4 * 4);
    }
    for (int i = tid; i < CHUNK * GDN_D / 4; i += GC_THREADS) {
      const int r = i / (GDN_D / 4), c4 = i % (GDN_D / 4);
      *reinterpret_cast<float4*>(wf + r * GC_PITCH + c4 * 4) =
          *reinterpret_cast<const float4*>(w + (ch * CHUNK + r) * GDN_D + c4 * 4);
    }
    for (int i = tid; i < CHUNK * GDN_D; i += GC_THREADS) {
      const int r = i / GDN_D, cc = i % GDN_D;
      const int64_t t = static_cast<int64_t>(c) * CHUNK + r;
      kf[r * GC_PITCH + cc] = t < token_num ? __bfloat162float(k[(tok_base + t) * k_t + h * k_h + cc]) : 0.f;
    }
    if (tid < CHUNK) gs[tid] = g_cumsum[ch * CHUNK + tid];
    __syncthreads();
    const float g_last = gs[CHUNK - 1];
    if (tid < CHUNK) dec[tid] = (c * CHUNK + tid < token_num) ? expf(g_last - gs[tid]) : 0.f;
    // delta[t][v] = u[t][v] - sum_k w[t][k] S[k][v]: thread = (t, 4 columns)
    {
      const int t = tid >> 2, c4 = (tid & 3) * 4;
      float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
      const float* wr = wf + t * GC_PITCH;
#pragma unroll 8
      for (int kk = 0; kk < GDN_D; ++kk) {
        const float a = wr[kk];
        const float4 s4 = *reinterpret_cast<const float4*>(st + kk * CS_BV + c4);
        a0 = fmaf(a, s4.x, a0);
        a1 = fmaf(a, s4.y, a1);
        a2 = fmaf(a, s4.z, a2);
        a3 = fmaf(a, s4.w, a3);
      }
      const float4 u4 = *reinterpret_cast<const float4*>(u_base + (ch * CHUNK + t) * GDN_D + v0 + c4);
      const float4 d4 = make_float4(u4.x - a0, u4.y - a1, u4.z - a2, u4.w - a3);
      *reinterpret_cast<float4*>(delta + (ch * CHUNK + t) * GDN_D + v0 + c4) = d4;
      *reinterpret_cast<float4*>(dl + t * CS_BV + c4) = d4;
    }
    __syncthreads();
    for (int i = tid; i < CHUNK * CS_BV; i += GC_THREADS) de[i] = dl[i] * dec[i / CS_BV];
    __syncthreads();
    // S[k][v] = exp(G_last) S[k][v] + sum_t k[t][k] de[t][v]: thread = (k, 8 columns)
    {
      const int kk = tid >> 1, c8 = (tid & 1) * 8;
      float acc[8];
      const float eg = expf(g_last);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = eg * st[kk * CS_BV + c8 + j];
#pragma unroll 4
      for (int t = 0; t < CHUNK; ++t) {
        const float a = kf[t * GC_PITCH + kk];
        const float4 x = *reinterpret_cast<const float4*>(de + t * CS_BV + c8);
        const float4 y = *reinterpret_cast<const float4*>(de + t * CS_BV + c8 + 4);
        acc[0] = fmaf(a, x.x, acc[0]); acc[1] = fmaf(a, x.y, acc[1]); acc[2] = fmaf(a, x.z, acc[2]); acc[3] = fmaf(a, x.w, acc[3]);
        acc[4] = fmaf(a, y.x, acc[4]); acc[5] = fmaf(a, y.y, acc[5]); acc[6] = fmaf(a, y.z, acc[6]); acc[7] = fmaf(a, y.w, acc[7]);
      }
      __syncthreads();  // every thread has read the old state
#pragma unroll
      for (int j = 0; j < 8; ++j) st[kk * CS_BV + c8 + j] = acc[j];
    }
    __syncthreads();
  }
  for (int i = tid; i < GDN_D * CS_BV / 4; i += GC_THREADS) {
    const int kk = i / (CS_BV / 4), q4 = i % (CS_BV / 4);
    *reinterpret_cast<float4*>(final_state + ((static_cast<int64_t>(blockIdx.z) * heads + h) * GDN_D + kk) * GDN_D + v0 +
                               q4 * 4) =
        *reinterpret_cast<const float4*>(st + kk * CS_BV + q4 * 4);
  }
}

// ---------------------------------------------------------------------------------------------------- chunk_output
constexpr int CO_SMEM = (2 * CHUNK * GC_PITCH + CHUNK * GC_LP + GDN_D * GC_PITCH + 2 * CHUNK) * 4;

__global__ void __launch_bounds__(GC_THREADS)
gdn_chunk_output_kernel(const __nv_bfloat16* __restrict__ q, int64_t q_t, int64_t q_h,
                        const __nv_bfloat16* __restrict__ k, int64_t k_t, int64_t k_h, const float* __restrict__ delta,
                        const float* __restrict__ g_cumsum, const float* __restrict__ chunk_state,
                        __nv_bfloat16* __restrict__ out, int64_t o_t, int64_t o_h, int token_num, int heads,
                        const int32_t* __restrict__ cu_seqlens) {
  extern __shared__ __align__(16) float sm[];
  const ChunkPos pos = locate_chunk(cu_seqlens, token_num);
  if (!pos.valid) return;
  token_num = pos.t_end;
  float* qf = sm;                           // [64][GC_PITCH]
  float* kd = qf + CHUNK * GC_PITCH;        // k, later delta [64][GC_PITCH]
  float* att = kd + CHUNK * GC_PITCH;       // [64][GC_LP]
  float* sf = att + CHUNK * GC_LP;          // state_in [128][GC_PITCH]
  float* gs = sf + GDN_D * GC_PITCH;        // G
  float* es = gs + CHUNK;                   // exp(G)
  const int chunk = pos.chunk, h = blockIdx.y, tid = threadIdx.x;
  const int t0 = pos.t0;
  const int64_t ch = static_cast<int64_t>(chunk) * heads + h;

  for (int i = tid; i < CHUNK * GDN_D; i += GC_THREADS) {
    const int r = i / GDN_D, c = i % GDN_D;
    const int64_t t = t0 + r;
    const bool ok = t < token_num;
    qf[r * GC_PITCH + c] = ok ? __bfloat162float(q[t * q_t + h * q_h + c]) : 0.f;
    kd[r * GC_PITCH + c] = ok ? __bfloat162float(k[t * k_t + h * k_h + c]) : 0.f;
  }
  for (int i = tid; i < GDN_D * GDN_D / 4; i += GC_THREADS) {
    const int r = i / (GDN_D / 4), c4 = i % (GDN_D / 4);
    *reinterpret_cast<float4*>(sf + r * GC_PITCH + c4 * 4) =
        *reinterpret_cast<const float4*>(chunk_state + (ch * GDN_D + r) * GDN_D + c4 * 4);
  }
  if (tid < CHUNK) {
    gs[tid] = g_cumsum[ch * CHUNK + tid];
    es[tid] = expf(gs[tid]);
  }
  __syncthreads();
  // ---- att[t][i] = <q_t, k_i> exp(G_t - G_i) for i <= t, both tokens valid
  {
    const int t = tid >> 2, ig = (tid & 3) * 16;
    const float4* qt = reinterpret_cast<const float4*>(qf + t * GC_PITCH);
    for (int ii = 0; ii < 16; ++ii) {
      const int i = ig + ii;
      float val = 0.f;
      if (i <= t && t0 + t < token_num) {
        const float4* ki = reinterpret_cast<const float4*>(kd + i * GC_PITCH);
        float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll 8
        for (int d = 0; d < GDN_D / 4; ++d) {
          const float4 x = qt[d], y = ki[d];
          a0 = fmaf(x.x, y.x, a0);
          a1 = fmaf(x.y, y.y, a1);
          a2 = fmaf(x.z, y.z, a2);
          a3 = fmaf(x.w, y.w, a3);
        }
        val = ((a0 + a1) + (a2 + a3)) * expf(gs[t] - gs[i]);
      }
      att[t * GC_LP + i] = val;
    }
  }
  __syncthreads();
  // k is no longer needed: its buffer takes delta
  for (int i = tid; i < CHUNK * GDN_D / 4; i += GC_THREADS) {
    const int r = i / (GDN_D / 4), c4 = i % (GDN_D / 4);
    *reinterpret_cast<float4*>(kd + r * GC_PITCH + c4 * 4) =
        *reinterpret_cast<const float4*>(delta + (ch * CHUNK + r) * GDN_D + c4 * 4);
  }
  __syncthreads();
  // ---- out = exp(G) (q @ S_in) + att @ delta : warp = 8 rows, lane = 4 columns
  {
    const int r0 = (tid >> 5) * 8, c0 = (tid & 31) * 4;
    float acc[8][4];
#pragma unroll
    for (int r = 0; r < 8; ++r) acc[r][0] = acc[r][1] = acc[r][2] = acc[r][3] = 0.f;
    for (int kk = 0; kk < GDN_D; ++kk) {
      const float4 b = *reinterpret_cast<const float4*>(sf + kk * GC_PITCH + c0);
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        const float a = qf[(r0 + r) * GC_PITCH + kk];
        acc[r][0] = fmaf(a, b.x, acc[r][0]);
        acc[r][1] = fmaf(a, b.y, acc[r][1]);
        acc[r][2] = fmaf(a, b.z, acc[r][2]);
        acc[r][3] = fmaf(a, b.w, acc[r][3]);
      }
    }
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      const float e = es[r0 + r];
      acc[r][0] *= e; acc[r][1] *= e; acc[r][2] *= e; acc[r][3] *= e;
    }
    for (int i = 0; i < r0 + 8; ++i) {  // att is lower triangular
      const float4 b = *reinterpret_cast<const float4*>(kd + i * GC_PITCH + c0);
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        const float a = att[(r0 + r) * GC_LP + i];
        acc[r][0] = fmaf(a, b.x, acc[r][0]);
        acc[r][1] = fmaf(a, b.y, acc[r][1]);
        acc[r][2] = fmaf(a, b.z, acc[r][2]);
        acc[r][3] = fmaf(a, b.w, acc[r][3]);
      }
    }
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      const int64_t t = t0 + r0 + r;
      if (t < token_num)
        *reinterpret_cast<uint2*>(out + t * o_t + h * o_h + c0) =
            make_uint2(pack_bf16(acc[r][0], acc[r][1]), pack_bf16(acc[r][2], acc[r][3]));
    }
  }
}

template <typename K>
static int set_smem(K kernel, int bytes, bool* flag_per_device, const char* what) {
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !flag_per_device[dev]) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess)
      return fail(ERR_RUNTIME, "%s: cannot raise dynamic shared memory to %d", what, bytes);
    flag_per_device[dev] = true;
  }
  return OK;
}

}  // namespace b200

using namespace b200;

extern "C" int b200_gdn_chunk_prepare_wy(const void* k, int64_t k_stride_t, int64_t k_stride_h, const void* v,
                                         int64_t v_stride_t, int64_t v_stride_h, const float* beta,
                                         int64_t beta_stride_t, int64_t beta_stride_h, const float* g,
                                         int64_t g_stride_t, int64_t g_stride_h, float* w, float* u_base,
                                         float* g_cumsum, int32_t token_num, int32_t num_heads, int32_t key_dim,
                                         int32_t value_dim, b200_stream_t stream) {
  B200_REQUIRE(token_num > 0 && num_heads > 0 && num_heads <= 65535, "gdn_chunk_prepare_wy: bad shape");
  B200_REQUIRE(key_dim == GDN_D && value_dim == GDN_D, "gdn_chunk_prepare_wy: key/value dim must be %d (got %d/%d)",
               GDN_D, key_dim, value_dim);
  static bool configured[64] = {false};
  int rc = set_smem(gdn_chunk_prepare_wy_kernel, PW_SMEM, configured, "gdn_chunk_prepare_wy");
  if (rc != OK) return rc;
  const int chunks = (token_num + CHUNK - 1) / CHUNK;
  gdn_chunk_prepare_wy_kernel<<<dim3(chunks, num_heads), GC_THREADS, PW_SMEM, reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(k), k_stride_t, k_stride_h, static_cast<const __nv_bfloat16*>(v), v_stride_t,
      v_stride_h, beta, beta_stride_t, beta_stride_h, g, g_stride_t, g_stride_h, w, u_base, g_cumsum, token_num,
      num_heads, nullptr);
  return check_launch("gdn_chunk_prepare_wy");
}

extern "C" int b200_gdn_chunk_state(const void* k, int64_t k_stride_t, int64_t k_stride_h, const float* w,
                                    const float* u_base, const float* g_cumsum, float* delta, float* chunk_state,
                                    float* final_state, int32_t token_num, int32_t num_heads, int32_t key_dim,
                                    int32_t value_dim, b200_stream_t stream) {
  B200_REQUIRE(token_num > 0 && num_heads > 0, "gdn_chunk_state: bad shape");
  B200_REQUIRE(key_dim == GDN_D && value_dim == GDN_D, "gdn_chunk_state: key/value dim must be %d (got %d/%d)", GDN_D,
               key_dim, value_dim);
  static bool configured[64] = {false};
  int rc = set_smem(gdn_chunk_state_kernel, CS_SMEM, configured, "gdn_chunk_state");
  if (rc != OK) return rc;
  const int chunks = (token_num + CHUNK - 1) / CHUNK;
  gdn_chunk_state_kernel<<<dim3(num_heads, GDN_D / CS_BV), GC_THREADS, CS_SMEM, reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(k), k_stride_t, k_stride_h, w, u_base, g_cumsum, delta, chunk_state,
      final_state, token_num, chunks, num_heads, nullptr);
  return check_launch("gdn_chunk_state");
}

extern "C" int b200_gdn_chunk_output(const void* q, int64_t q_stride_t, int64_t q_stride_h, const void* k,
                                     int64_t k_stride_t, int64_t k_stride_h, const float* delta, const float* g_cumsum,
                                     const float* chunk_state, void* out, int64_t out_stride_t, int64_t out_stride_h,
                                     int32_t token_num, int32_t num_heads, int32_t key_dim, int32_t value_dim,
                                     b200_stream_t stream) {
  B200_REQUIRE(token_num > 0 && num_heads > 0 && num_heads <= 65535, "gdn_chunk_output: bad shape");
  B200_REQUIRE(key_dim == GDN_D && value_dim == GDN_D, "gdn_chunk_output: key/value dim must be %d (got %d/%d)", GDN_D,
               key_dim, value_dim);
  B200_REQUIRE((reinterpret_cast<uintptr_t>(out) % 8 == 0) && out_stride_t % 4 == 0 && out_stride_h % 4 == 0,
               "gdn_chunk_output: out must be 8-byte aligned with strides that are multiples of 4");
  static bool configured[64] = {false};
  int rc = set_smem(gdn_chunk_output_kernel, CO_SMEM, configured, "gdn_chunk_output");
  if (rc != OK) return rc;
  const int chunks = (token_num + CHUNK - 1) / CHUNK;
  gdn_chunk_output_kernel<<<dim3(chunks, num_heads), GC_THREADS, CO_SMEM, reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(q), q_stride_t, q_stride_h, static_cast<const __nv_bfloat16*>(k), k_stride_t,
      k_stride_h, delta, g_cumsum, chunk_state, static_cast<__nv_bfloat16*>(out), out_stride_t, out_stride_h, token_num,
      num_heads, nullptr);
  return check_launch("gdn_chunk_output");
}

// Packed chunk-64 prefill: the three stages over a batch of sequences packed in one buffer, chunk grid restarting at
// every cu_seqlens[b], zero state at each sequence start.  The reference has no such call (its chunk path is
// single-sequence, engine/runner.py:263-267); it is the packed form a batched prefill (32 prompts in one buffer) needs.
// Workspace layout (fp32): w | u_base | delta [Nmax,H,64,128] each, g_cumsum [Nmax,H,64], chunk_state [Nmax,H,128,128]
// with Nmax = total_tokens / 64 + batch (an upper bound of the number of chunks that needs no device read).
extern "C" int64_t b200_gdn_chunked_prefill_packed_workspace_bytes(int32_t batch, int32_t total_tokens, int32_t num_heads) {
  const int64_t n = static_cast<int64_t>(total_tokens) / CHUNK + batch;
  return n * num_heads * (3LL * CHUNK * GDN_D + CHUNK + static_cast<int64_t>(GDN_D) * GDN_D) * 4;
}

extern "C" int b200_gdn_chunked_prefill_packed(const void* q, int64_t q_stride_t, int64_t q_stride_h, const void* k,
                                               int64_t k_stride_t, int64_t k_stride_h, const void* v,
                                               int64_t v_stride_t, int64_t v_stride_h, const float* beta,
                                               int64_t beta_stride_t, int64_t beta_stride_h, const float* g,
                                               int64_t g_stride_t, int64_t g_stride_h, const int32_t* cu_seqlens,
                                               int32_t batch, int32_t total_tokens, int32_t max_seqlen, void* workspace,
                                               float* state, void* out, int64_t out_stride_t, int64_t out_stride_h,
                                               int32_t num_heads, int32_t key_dim, int32_t value_dim,
                                               b200_stream_t stream) {
  B200_REQUIRE(batch > 0 && batch <= 65535 && total_tokens > 0 && num_heads > 0 && num_heads <= 65535,
               "gdn_chunked_prefill_packed: bad shape");
  B200_REQUIRE(key_dim == GDN_D && value_dim == GDN_D,
               "gdn_chunked_prefill_packed: key/value dim must be %d (got %d/%d)", GDN_D, key_dim, value_dim);
  B200_REQUIRE(cu_seqlens != nullptr && workspace != nullptr && aligned16(workspace),
               "gdn_chunked_prefill_packed: cu_seqlens and a 16-byte aligned workspace are required");
  B200_REQUIRE((reinterpret_cast<uintptr_t>(out) % 8 == 0) && out_stride_t % 4 == 0 && out_stride_h % 4 == 0,
               "gdn_chunked_prefill_packed: out must be 8-byte aligned with strides that are multiples of 4");
  if (max_seqlen <= 0) return OK;
  static bool c1[64] = {false}, c2[64] = {false}, c3[64] = {false};
  int rc = set_smem(gdn_chunk_prepare_wy_kernel, PW_SMEM, c1, "gdn_chunked_prefill_packed");
  if (rc == OK) rc = set_smem(gdn_chunk_state_kernel, CS_SMEM, c2, "gdn_chunked_prefill_packed");
  if (rc == OK) rc = set_smem(gdn_chunk_output_kernel, CO_SMEM, c3, "gdn_chunked_prefill_packed");
  if (rc != OK) return rc;
  const int64_t n = static_cast<int64_t>(total_tokens) / CHUNK + batch;
  float* w = static_cast<float*>(workspace);
  float* u = w + n * num_heads * CHUNK * GDN_D;
  float* delta = u + n * num_heads * CHUNK * GDN_D;
  float* gcs = delta + n * num_heads * CHUNK * GDN_D;
  float* cstate = gcs + n * num_heads * CHUNK;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int chunks = (max_seqlen + CHUNK - 1) / CHUNK;
  const __nv_bfloat16* qb = static_cast<const __nv_bfloat16*>(q);
  const __nv_bfloat16* kb = static_cast<const __nv_bfloat16*>(k);
  const __nv_bfloat16* vb = static_cast<const __nv_bfloat16*>(v);
  gdn_chunk_prepare_wy_kernel<<<dim3(chunks, num_heads, batch), GC_THREADS, PW_SMEM, st>>>(
      kb, k_stride_t, k_stride_h, vb, v_stride_t, v_stride_h, beta, beta_stride_t, beta_stride_h, g, g_stride_t,
      g_stride_h, w, u, gcs, total_tokens, num_heads, cu_seqlens);
  rc = check_launch("gdn_chunked_prefill_packed (prepare_wy)");
  if (rc != OK) return rc;
  gdn_chunk_state_kernel<<<dim3(num_heads, GDN_D / CS_BV, batch), GC_THREADS, CS_SMEM, st>>>(
      kb, k_stride_t, k_stride_h, w, u, gcs, delta, cstate, state, total_tokens, chunks, num_heads, cu_seqlens);
  rc = check_launch("gdn_chunked_prefill_packed (state)");
  if (rc != OK) return rc;
  gdn_chunk_output_kernel<<<dim3(chunks, num_heads, batch), GC_THREADS, CO_SMEM, st>>>(
      qb, q_stride_t, q_stride_h, kb, k_stride_t, k_stride_h, delta, gcs, cstate, static_cast<__nv_bfloat16*>(out),
      out_stride_t, out_stride_h, total_tokens, num_heads, cu_seqlens);
  return check_launch("gdn_chunked_prefill_packed (output)");
}
