// Gated-DeltaNet chunk-64 prefill as the reference's three operators, with its intermediate tensors:
//   b200_gdn_chunk_prepare_wy <-> triton_kernels/gdn_recurrent_prefill.py:703-784 (kernel :248-396)
//   b200_gdn_chunk_state      <-> triton_kernels/gdn_recurrent_prefill.py:825-909 (kernel :404-537)
//   b200_gdn_chunk_output     <-> triton_kernels/gdn_recurrent_prefill.py:935-1006 (kernel :563-690)
// Per chunk (G = cumsum(g) inside the chunk, S_in the state entering it):
//   L[t,i] = beta_t exp(G_t - G_i) <k_t,k_i> (i<t);  P = (I+L)^-1;  u = P (beta v);  w = P (beta exp(G) k)
//   delta = u - w S_in;  S_out = exp(G_last) S_in + sum_t k_t (exp(G_last - G_t) delta_t)^T
//   o_t = exp(G_t) q_t^T S_in + sum_{i<=t} <q_t,k_i> exp(G_t - G_i) delta_i
// The products run on the tensor cores (mma.sync m16n8k16, bf16 inputs, fp32 accumulation): exact bf16 operands for
// k k^T and q k^T, bf16 pairs hi + lo for every fp32 operand (the reference holds its 5e-4 state tolerance with 3xTF32
// products of the same accuracy); only the 64 x 64 triangular inverse stays on the CUDA cores.  These kernels keep the
// reference's data flow through HBM so that each operator can be swapped individually.
#include "b200_attn.h"
#include "common.cuh"
#include "gdn_inverse.cuh"

namespace b200 {

constexpr int GC_THREADS = 256;
constexpr int GC_LP = INV_LP;         // fp32 pitch of the [64][64] L and inverse tiles

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

// ------------------------------------------------------------------------------------------- tensor-core plumbing
// Every product below is mma.sync m16n8k16 (bf16 inputs, fp32 accumulation) on bf16 tiles in shared memory.  q, k and v
// are bf16 already, so a product of two of them is exact up to the fp32 accumulation; an fp32 operand (the inverse, w,
// delta, the state, the decayed attention) is fed as a bf16 pair hi + lo with the cross products hi*hi + hi*lo + lo*hi
// (hi*hi + lo*hi when the other operand is exact), about 16 mantissa bits per factor - the order of the reference's
// 3xTF32 products.
constexpr int GC_P128 = GDN_D + 8;  // bf16 pitch of [rows][128] tiles: 272-byte rows, conflict-free fragment loads
constexpr int GC_P64 = CHUNK + 8;   // bf16 pitch of [rows][64] tiles

__device__ __forceinline__ uint32_t ld_pair(const __nv_bfloat16* p) { return *reinterpret_cast<const uint32_t*>(p); }
__device__ __forceinline__ void split_pair(float x0, float x1, uint32_t& hi, uint32_t& lo) {
  const __nv_bfloat16 h0 = __float2bfloat16_rn(x0), h1 = __float2bfloat16_rn(x1);
  hi = static_cast<uint32_t>(__bfloat16_as_ushort(h0)) | (static_cast<uint32_t>(__bfloat16_as_ushort(h1)) << 16);
  lo = pack_bf16(x0 - __bfloat162float(h0), x1 - __bfloat162float(h1));
}
// A fragment (rows m0..m0+15, k0..k0+15) of a tile stored [M][K], K contiguous
__device__ __forceinline__ void frag_a(uint32_t (&a)[4], const __nv_bfloat16* A, int pitch, int m0, int k0, int lane) {
  const __nv_bfloat16* p = A + (m0 + (lane >> 2)) * pitch + k0 + (lane & 3) * 2;
  a[0] = ld_pair(p);
  a[1] = ld_pair(p + 8 * pitch);
  a[2] = ld_pair(p + 8);
  a[3] = ld_pair(p + 8 * pitch + 8);
}
// A fragment of A = T^T for a tile T stored [K][M], M contiguous (transposing ldmatrix)
__device__ __forceinline__ void frag_a_t(uint32_t (&a)[4], const __nv_bfloat16* T, int pitch, int m0, int k0, int lane) {
  const int j = lane >> 3, r = lane & 7;
  ldmatrix_x4_trans(a, smem_u32(T + (k0 + (j >> 1) * 8 + r) * pitch + m0 + (j & 1) * 8));
}
// B fragment (k0..k0+15, columns n0..n0+7) of a tile stored [N][K], K contiguous
__device__ __forceinline__ void frag_b_nk(uint32_t (&b)[2], const __nv_bfloat16* Bt, int pitch, int n0, int k0, int lane) {
  const __nv_bfloat16* p = Bt + (n0 + (lane >> 2)) * pitch + k0 + (lane & 3) * 2;
  b[0] = ld_pair(p);
  b[1] = ld_pair(p + 8);
}
// B fragments of the two column tiles n0..n0+7 (b[0], b[1]) and n0+8..n0+15 (b[2], b[3]) of a tile stored [K][N],
// N contiguous (transposing ldmatrix)
__device__ __forceinline__ void frag_b_kn(uint32_t (&b)[4], const __nv_bfloat16* B, int pitch, int k0, int n0, int lane) {
  const int j = lane >> 3, r = lane & 7;
  ldmatrix_x4_trans(b, smem_u32(B + (k0 + (j & 1) * 8 + r) * pitch + n0 + (j >> 1) * 8));
}

// 64 rows x 128 bf16 of one head from a strided [T, H, 128] activation into a [64][GC_P128] tile; rows from `t_end` on
// are zero.  16-byte loads when the row addresses allow it.
__device__ __forceinline__ void load_rows_bf16(__nv_bfloat16* tile, const __nv_bfloat16* src, int64_t stride_t, int64_t t0,
                                               int64_t t_end, int tid) {
  const bool vec = (reinterpret_cast<uintptr_t>(src) & 15) == 0 && (stride_t & 7) == 0;
  if (vec) {
    for (int i = tid; i < CHUNK * (GDN_D / 8); i += GC_THREADS) {
      const int r = i >> 4, c8 = (i & 15) * 8;
      uint4 val = make_uint4(0, 0, 0, 0);
      if (t0 + r < t_end) val = *reinterpret_cast<const uint4*>(src + (t0 + r) * stride_t + c8);
      *reinterpret_cast<uint4*>(tile + r * GC_P128 + c8) = val;
    }
  } else {
    for (int i = tid; i < CHUNK * GDN_D; i += GC_THREADS) {
      const int r = i >> 7, c = i & 127;
      tile[r * GC_P128 + c] = t0 + r < t_end ? src[(t0 + r) * stride_t + c] : __float2bfloat16_rn(0.f);
    }
  }
}
// C[64 x 64] = X K^T over the 128 dims for the column tiles that can hold a causal entry (column <= row): warp =
// (16-row tile mt, 32-column half nh); acc[nt] is the 16 x 8 tile at columns nh*32 + nt*8.
__device__ __forceinline__ void causal_scores(float (&acc)[4][4], const __nv_bfloat16* X, const __nv_bfloat16* K, int mt,
                                              int nh, int lane) {
#pragma unroll
  for (int nt = 0; nt < 4; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
  if (nh * 32 > mt * 16 + 15) return;
#pragma unroll
  for (int ks = 0; ks < GDN_D / 16; ++ks) {
    uint32_t a[4];
    frag_a(a, X, GC_P128, mt * 16, ks * 16, lane);
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      if (nh * 32 + nt * 8 > mt * 16 + 15) continue;
      uint32_t b[2];
      frag_b_nk(b, K, GC_P128, nh * 32 + nt * 8, ks * 16, lane);
      mma_bf16_16816(acc[nt], a, b[0], b[1]);
    }
  }
}

// ---------------------------------------------------------------------------------------------------- prepare_wy
// shared memory: k, v tiles (bf16) | lower, inv (fp32) | (inv beta) and (inv beta e^G) as bf16 pairs | scalars
constexpr int PW_KB = 0;
constexpr int PW_VB = PW_KB + CHUNK * GC_P128 * 2;
constexpr int PW_LOWER = PW_VB + CHUNK * GC_P128 * 2;
constexpr int PW_INV = PW_LOWER + CHUNK * GC_LP * 4;
constexpr int PW_PAIR = PW_INV + CHUNK * GC_LP * 4;      // four [64][GC_P64] bf16 tiles; first the inverse's scratch
constexpr int PW_SC = PW_PAIR + 4 * CHUNK * GC_P64 * 2;
static_assert(INV_SCRATCH_FLOATS * 4 <= 4 * CHUNK * GC_P64 * 2, "the merge scratch lies over the pair tiles");
constexpr int PW_SMEM = PW_SC + 3 * CHUNK * 4;

__global__ void __launch_bounds__(GC_THREADS)
gdn_chunk_prepare_wy_kernel(const __nv_bfloat16* __restrict__ k, int64_t k_t, int64_t k_h,
                            const __nv_bfloat16* __restrict__ v, int64_t v_t, int64_t v_h,
                            const float* __restrict__ beta, int64_t be_t, int64_t be_h, const float* __restrict__ g,
                            int64_t g_t, int64_t g_h, float* __restrict__ w, float* __restrict__ u_base,
                            float* __restrict__ g_cumsum, int token_num, int heads,
                            const int32_t* __restrict__ cu_seqlens) {
  extern __shared__ __align__(16) uint8_t smem_pw[];
  const ChunkPos pos = locate_chunk(cu_seqlens, token_num);
  if (!pos.valid) return;
  token_num = pos.t_end;
  __nv_bfloat16* kb = reinterpret_cast<__nv_bfloat16*>(smem_pw + PW_KB);   // [64][GC_P128]
  __nv_bfloat16* vb = reinterpret_cast<__nv_bfloat16*>(smem_pw + PW_VB);   // [64][GC_P128]
  float* lower = reinterpret_cast<float*>(smem_pw + PW_LOWER);             // [64][GC_LP]
  float* inv = reinterpret_cast<float*>(smem_pw + PW_INV);                 // [64][GC_LP]
  __nv_bfloat16* pu_hi = reinterpret_cast<__nv_bfloat16*>(smem_pw + PW_PAIR);  // inv[t][i] beta_i
  __nv_bfloat16* pu_lo = pu_hi + CHUNK * GC_P64;
  __nv_bfloat16* pw_hi = pu_lo + CHUNK * GC_P64;                               // inv[t][i] beta_i e^{G_i}
  __nv_bfloat16* pw_lo = pw_hi + CHUNK * GC_P64;
  float* gs = reinterpret_cast<float*>(smem_pw + PW_SC);  // g, then G
  float* bs = gs + CHUNK;                                 // beta
  float* es = bs + CHUNK;                                 // exp(G)
  const int chunk = pos.chunk, h = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int t0 = pos.t0;

  load_rows_bf16(kb, k + h * k_h, k_t, t0, token_num, tid);
  load_rows_bf16(vb, v + h * v_h, v_t, t0, token_num, tid);
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
  // ---- lower[t][i] = beta_t exp(G_t - G_i) <k_t, k_i> for i < t, both tokens valid (k k^T on the tensor cores)
  const int mt = warp & 3, nh = warp >> 2, gr = lane >> 2, tg = (lane & 3) * 2;
  {
    float acc[4][4];
    causal_scores(acc, kb, kb, mt, nh, lane);
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int t = mt * 16 + gr + (e >> 1) * 8, i = nh * 32 + nt * 8 + tg + (e & 1);
        lower[t * GC_LP + i] = (i < t && t0 + t < token_num) ? bs[t] * expf(gs[t] - gs[i]) * acc[nt][e] : 0.f;
      }
  }
  __syncthreads();
  // ---- inv = (I + lower)^-1, blocked, by the first four warps (blocks above the block diagonal are not written)
  if (tid < 128) blocked_inverse64(lower, inv, reinterpret_cast<float*>(smem_pw + PW_PAIR), tid);
  __syncthreads();
  // ---- the right-hand scalings move into the inverse: u = (inv diag(beta)) v, w = (inv diag(beta e^G)) k, so that the
  //      right operands stay the exact bf16 inputs
  for (int idx = tid; idx < CHUNK * CHUNK / 2; idx += GC_THREADS) {
    const int t = idx >> 5, i = (idx & 31) * 2;
    const float p0 = i <= t ? inv[t * GC_LP + i] * bs[i] : 0.f;
    const float p1 = i + 1 <= t ? inv[t * GC_LP + i + 1] * bs[i + 1] : 0.f;
    uint32_t hi, lo;
    split_pair(p0, p1, hi, lo);
    *reinterpret_cast<uint32_t*>(pu_hi + t * GC_P64 + i) = hi;
    *reinterpret_cast<uint32_t*>(pu_lo + t * GC_P64 + i) = lo;
    split_pair(p0 * es[i], p1 * es[i + 1], hi, lo);
    *reinterpret_cast<uint32_t*>(pw_hi + t * GC_P64 + i) = hi;
    *reinterpret_cast<uint32_t*>(pw_lo + t * GC_P64 + i) = lo;
  }
  __syncthreads();
  // ---- u and w: warp = (16-row tile mt, 64-column half nh); inv is lower triangular, so k steps past the row tile
  //      contribute nothing
  const int64_t out_base = (static_cast<int64_t>(chunk) * heads + h) * CHUNK * GDN_D;
#pragma unroll
  for (int which = 0; which < 2; ++which) {
    const __nv_bfloat16* a_hi = which == 0 ? pu_hi : pw_hi;
    const __nv_bfloat16* a_lo = which == 0 ? pu_lo : pw_lo;
    const __nv_bfloat16* rhs = which == 0 ? vb : kb;
    float acc[8][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
    for (int ks = 0; ks <= mt; ++ks) {
      uint32_t ah[4], al[4];
      frag_a(ah, a_hi, GC_P64, mt * 16, ks * 16, lane);
      frag_a(al, a_lo, GC_P64, mt * 16, ks * 16, lane);
#pragma unroll
      for (int np = 0; np < 4; ++np) {
        uint32_t b[4];
        frag_b_kn(b, rhs, GC_P128, ks * 16, nh * 64 + np * 16, lane);
        mma_bf16_16816(acc[2 * np], ah, b[0], b[1]);
        mma_bf16_16816(acc[2 * np], al, b[0], b[1]);
        mma_bf16_16816(acc[2 * np + 1], ah, b[2], b[3]);
        mma_bf16_16816(acc[2 * np + 1], al, b[2], b[3]);
      }
    }
    float* dst = (which == 0 ? u_base : w) + out_base;
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      const int c = nh * 64 + nt * 8 + tg;
      *reinterpret_cast<float2*>(dst + (mt * 16 + gr) * GDN_D + c) = make_float2(acc[nt][0], acc[nt][1]);
      *reinterpret_cast<float2*>(dst + (mt * 16 + gr + 8) * GDN_D + c) = make_float2(acc[nt][2], acc[nt][3]);
    }
  }
}

// ---------------------------------------------------------------------------------------------------- chunk_state
constexpr int CS_BV = 32;           // value columns per CTA
constexpr int GC_PV = CS_BV + 8;    // bf16 pitch of [rows][CS_BV] tiles
// shared memory: w pair [64][GC_P128] x 2 | k [64][GC_P128] | state pair [128][GC_PV] x 2 | decayed delta pair
// [64][GC_PV] x 2 | G, decay
constexpr int CS_WH = 0;
constexpr int CS_WL = CS_WH + CHUNK * GC_P128 * 2;
constexpr int CS_KB = CS_WL + CHUNK * GC_P128 * 2;
constexpr int CS_SH = CS_KB + CHUNK * GC_P128 * 2;
constexpr int CS_SL = CS_SH + GDN_D * GC_PV * 2;
constexpr int CS_DH = CS_SL + GDN_D * GC_PV * 2;
constexpr int CS_DL = CS_DH + CHUNK * GC_PV * 2;
constexpr int CS_SC = CS_DL + CHUNK * GC_PV * 2;
constexpr int CS_SMEM = CS_SC + 2 * CHUNK * 4;
constexpr int CS_W_PER_THREAD = CHUNK * GDN_D / 4 / GC_THREADS;  // float4 of w per thread and chunk (8)
constexpr int CS_K_PER_THREAD = CHUNK * GDN_D / 8 / GC_THREADS;  // 16-byte pieces of k per thread and chunk (4)

// The w and k rows of one chunk, fetched into registers one chunk ahead so that their latency hides behind the
// products of the chunk in front.
struct ChunkOperands {
  float4 w[CS_W_PER_THREAD];
  uint4 k[CS_K_PER_THREAD];
};
__device__ __forceinline__ void fetch_operands(ChunkOperands& r, const float* w_chunk, const __nv_bfloat16* k_head,
                                               int64_t k_t, int64_t t0, int64_t t_end, bool k_vec, int tid) {
#pragma unroll
  for (int j = 0; j < CS_W_PER_THREAD; ++j) {
    const int i = tid + j * GC_THREADS;
    r.w[j] = *reinterpret_cast<const float4*>(w_chunk + static_cast<int64_t>(i >> 5) * GDN_D + (i & 31) * 4);
  }
#pragma unroll
  for (int j = 0; j < CS_K_PER_THREAD; ++j) {
    const int i = tid + j * GC_THREADS, row = i >> 4, c8 = (i & 15) * 8;
    uint4 val = make_uint4(0, 0, 0, 0);
    if (t0 + row < t_end) {
      const __nv_bfloat16* src = k_head + (t0 + row) * k_t + c8;
      if (k_vec) {
        val = *reinterpret_cast<const uint4*>(src);
      } else {
        uint32_t u[4];
#pragma unroll
        for (int e = 0; e < 4; ++e)
          u[e] = static_cast<uint32_t>(__bfloat16_as_ushort(src[2 * e])) |
                 (static_cast<uint32_t>(__bfloat16_as_ushort(src[2 * e + 1])) << 16);
        val = make_uint4(u[0], u[1], u[2], u[3]);
      }
    }
    r.k[j] = val;
  }
}
__device__ __forceinline__ void stage_operands(const ChunkOperands& r, __nv_bfloat16* wh, __nv_bfloat16* wl,
                                               __nv_bfloat16* kb, int tid) {
#pragma unroll
  for (int j = 0; j < CS_W_PER_THREAD; ++j) {
    const int i = tid + j * GC_THREADS, row = i >> 5, c4 = (i & 31) * 4;
    uint32_t h0, l0, h1, l1;
    split_pair(r.w[j].x, r.w[j].y, h0, l0);
    split_pair(r.w[j].z, r.w[j].w, h1, l1);
    *reinterpret_cast<uint2*>(wh + row * GC_P128 + c4) = make_uint2(h0, h1);
    *reinterpret_cast<uint2*>(wl + row * GC_P128 + c4) = make_uint2(l0, l1);
  }
#pragma unroll
  for (int j = 0; j < CS_K_PER_THREAD; ++j) {
    const int i = tid + j * GC_THREADS;
    *reinterpret_cast<uint4*>(kb + (i >> 4) * GC_P128 + (i & 15) * 8) = r.k[j];
  }
}

// (capping the registers at 128 for two CTAs per SM was tried: 20 % faster on a packed batch, 50 % slower on the one
// long sequence this path is routed to)
__global__ void __launch_bounds__(GC_THREADS)
gdn_chunk_state_kernel(const __nv_bfloat16* __restrict__ k, int64_t k_t, int64_t k_h, const float* __restrict__ w,
                       const float* __restrict__ u_base, const float* __restrict__ g_cumsum, float* __restrict__ delta,
                       float* __restrict__ chunk_state, float* __restrict__ final_state, int token_num, int num_chunks,
                       int heads, const int32_t* __restrict__ cu_seqlens) {
  extern __shared__ __align__(16) uint8_t smem_cs[];
  // packed batch: blockIdx.z = sequence; its chunks are [chunk_base, chunk_base + num_chunks)
  int chunk_base = 0, tok_base = 0;
  if (cu_seqlens != nullptr) {
    const int b = blockIdx.z;
    for (int i = 0; i < b; ++i) chunk_base += (cu_seqlens[i + 1] - cu_seqlens[i] + CHUNK - 1) / CHUNK;
    tok_base = cu_seqlens[b];
    token_num = cu_seqlens[b + 1] - tok_base;
    num_chunks = (token_num + CHUNK - 1) / CHUNK;
  }
  __nv_bfloat16* wh = reinterpret_cast<__nv_bfloat16*>(smem_cs + CS_WH);
  __nv_bfloat16* wl = reinterpret_cast<__nv_bfloat16*>(smem_cs + CS_WL);
  __nv_bfloat16* kb = reinterpret_cast<__nv_bfloat16*>(smem_cs + CS_KB);
  __nv_bfloat16* sh = reinterpret_cast<__nv_bfloat16*>(smem_cs + CS_SH);
  __nv_bfloat16* sl = reinterpret_cast<__nv_bfloat16*>(smem_cs + CS_SL);
  __nv_bfloat16* dh = reinterpret_cast<__nv_bfloat16*>(smem_cs + CS_DH);
  __nv_bfloat16* dl = reinterpret_cast<__nv_bfloat16*>(smem_cs + CS_DL);
  float* gs = reinterpret_cast<float*>(smem_cs + CS_SC);  // G [64]
  float* dec = gs + CHUNK;                                // exp(G_last - G) (0 for padded tokens)
  const int h = blockIdx.x, v0 = blockIdx.y * CS_BV, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int gr = lane >> 2, tg = (lane & 3) * 2;
  const __nv_bfloat16* k_head = k + h * k_h;
  const bool k_vec = (reinterpret_cast<uintptr_t>(k_head) & 15) == 0 && (k_t & 7) == 0;
  const int64_t seq_end = static_cast<int64_t>(tok_base) + token_num;

  // the state slice [128 dk][32 dv] lives in accumulator registers: warp = key rows 16*warp .. +15, st[nt] = the
  // 16 x 8 tile at value columns nt*8
  float st[CS_BV / 8][4];
#pragma unroll
  for (int nt = 0; nt < CS_BV / 8; ++nt) st[nt][0] = st[nt][1] = st[nt][2] = st[nt][3] = 0.f;

  ChunkOperands ops_next;
  if (num_chunks > 0)
    fetch_operands(ops_next, w + (static_cast<int64_t>(chunk_base) * heads + h) * CHUNK * GDN_D, k_head, k_t, tok_base,
                   seq_end, k_vec, tid);
  for (int c = 0; c < num_chunks; ++c) {
    const int64_t ch = static_cast<int64_t>(chunk_base + c) * heads + h;
    // state entering the chunk: fp32 to global memory, bf16 pair to shared memory (right operand of w S)
#pragma unroll
    for (int nt = 0; nt < CS_BV / 8; ++nt)
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int kk = warp * 16 + gr + half * 8, col = nt * 8 + tg;
        const float s0 = st[nt][2 * half], s1 = st[nt][2 * half + 1];
        *reinterpret_cast<float2*>(chunk_state + (ch * GDN_D + kk) * GDN_D + v0 + col) = make_float2(s0, s1);
        uint32_t hi, lo;
        split_pair(s0, s1, hi, lo);
        *reinterpret_cast<uint32_t*>(sh + kk * GC_PV + col) = hi;
        *reinterpret_cast<uint32_t*>(sl + kk * GC_PV + col) = lo;
      }
    stage_operands(ops_next, wh, wl, kb, tid);
    if (tid < CHUNK) {
      const float gv = g_cumsum[ch * CHUNK + tid];
      const float g_last_v = g_cumsum[ch * CHUNK + CHUNK - 1];
      gs[tid] = gv;
      dec[tid] = (c * CHUNK + tid < token_num) ? expf(g_last_v - gv) : 0.f;
    }
    __syncthreads();
    if (c + 1 < num_chunks)
      fetch_operands(ops_next, w + (ch + heads) * CHUNK * GDN_D, k_head, k_t,
                     static_cast<int64_t>(tok_base) + static_cast<int64_t>(c + 1) * CHUNK, seq_end, k_vec, tid);
    const float g_last = gs[CHUNK - 1];
    // delta[t][v] = u[t][v] - sum_k w[t][k] S[k][v]: warp = (16-token tile mt, 16-column pair np)
    {
      const int mt = warp & 3, np = warp >> 2;
      float2 u2[2][2];
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int half = 0; half < 2; ++half)
          u2[nt][half] = *reinterpret_cast<const float2*>(u_base + (ch * CHUNK + mt * 16 + gr + half * 8) * GDN_D + v0 +
                                                          np * 16 + nt * 8 + tg);
      float acc[2][4];
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
#pragma unroll
      for (int ks = 0; ks < GDN_D / 16; ++ks) {
        uint32_t ah[4], al[4], bh[4], bl[4];
        frag_a(ah, wh, GC_P128, mt * 16, ks * 16, lane);
        frag_a(al, wl, GC_P128, mt * 16, ks * 16, lane);
        frag_b_kn(bh, sh, GC_PV, ks * 16, np * 16, lane);
        frag_b_kn(bl, sl, GC_PV, ks * 16, np * 16, lane);
        mma_bf16_16816(acc[0], ah, bh[0], bh[1]);
        mma_bf16_16816(acc[0], ah, bl[0], bl[1]);
        mma_bf16_16816(acc[0], al, bh[0], bh[1]);
        mma_bf16_16816(acc[1], ah, bh[2], bh[3]);
        mma_bf16_16816(acc[1], ah, bl[2], bl[3]);
        mma_bf16_16816(acc[1], al, bh[2], bh[3]);
      }
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int t = mt * 16 + gr + half * 8, col = np * 16 + nt * 8 + tg;
          const float d0 = u2[nt][half].x - acc[nt][2 * half], d1 = u2[nt][half].y - acc[nt][2 * half + 1];
          *reinterpret_cast<float2*>(delta + (ch * CHUNK + t) * GDN_D + v0 + col) = make_float2(d0, d1);
          uint32_t hi, lo;
          split_pair(d0 * dec[t], d1 * dec[t], hi, lo);
          *reinterpret_cast<uint32_t*>(dh + t * GC_PV + col) = hi;
          *reinterpret_cast<uint32_t*>(dl + t * GC_PV + col) = lo;
        }
    }
    __syncthreads();
    // S[k][v] = exp(G_last) S[k][v] + sum_t k[t][k] (delta[t][v] exp(G_last - G_t)): A = k^T through the transposing
    // ldmatrix, exact in bf16
    {
      const float eg = expf(g_last);
#pragma unroll
      for (int nt = 0; nt < CS_BV / 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) st[nt][e] *= eg;
#pragma unroll
      for (int ks = 0; ks < CHUNK / 16; ++ks) {
        uint32_t a[4];
        frag_a_t(a, kb, GC_P128, warp * 16, ks * 16, lane);
#pragma unroll
        for (int np = 0; np < CS_BV / 16; ++np) {
          uint32_t bh[4], bl[4];
          frag_b_kn(bh, dh, GC_PV, ks * 16, np * 16, lane);
          frag_b_kn(bl, dl, GC_PV, ks * 16, np * 16, lane);
          mma_bf16_16816(st[2 * np], a, bh[0], bh[1]);
          mma_bf16_16816(st[2 * np], a, bl[0], bl[1]);
          mma_bf16_16816(st[2 * np + 1], a, bh[2], bh[3]);
          mma_bf16_16816(st[2 * np + 1], a, bl[2], bl[3]);
        }
      }
    }
    __syncthreads();  // the tiles are rewritten by the next chunk
  }
#pragma unroll
  for (int nt = 0; nt < CS_BV / 8; ++nt)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int kk = warp * 16 + gr + half * 8, col = nt * 8 + tg;
      *reinterpret_cast<float2*>(final_state + ((static_cast<int64_t>(blockIdx.z) * heads + h) * GDN_D + kk) * GDN_D + v0 +
                                 col) = make_float2(st[nt][2 * half], st[nt][2 * half + 1]);
    }
}

// ---------------------------------------------------------------------------------------------------- chunk_output
// shared memory: q, k [64][GC_P128] | state pair [128][GC_P128] x 2 | delta pair [64][GC_P128] x 2 | attention pair
// [64][GC_P64] x 2 | G, exp(G)
constexpr int CO_QB = 0;
constexpr int CO_KB = CO_QB + CHUNK * GC_P128 * 2;
constexpr int CO_SH = CO_KB + CHUNK * GC_P128 * 2;
constexpr int CO_SL = CO_SH + GDN_D * GC_P128 * 2;
constexpr int CO_DH = CO_SL + GDN_D * GC_P128 * 2;
constexpr int CO_DL = CO_DH + CHUNK * GC_P128 * 2;
constexpr int CO_AH = CO_DL + CHUNK * GC_P128 * 2;
constexpr int CO_AL = CO_AH + CHUNK * GC_P64 * 2;
constexpr int CO_SC = CO_AL + CHUNK * GC_P64 * 2;
constexpr int CO_SMEM = CO_SC + 2 * CHUNK * 4;

__global__ void __launch_bounds__(GC_THREADS)
gdn_chunk_output_kernel(const __nv_bfloat16* __restrict__ q, int64_t q_t, int64_t q_h,
                        const __nv_bfloat16* __restrict__ k, int64_t k_t, int64_t k_h, const float* __restrict__ delta,
                        const float* __restrict__ g_cumsum, const float* __restrict__ chunk_state,
                        __nv_bfloat16* __restrict__ out, int64_t o_t, int64_t o_h, int token_num, int heads,
                        const int32_t* __restrict__ cu_seqlens) {
  extern __shared__ __align__(16) uint8_t smem_co[];
  const ChunkPos pos = locate_chunk(cu_seqlens, token_num);
  if (!pos.valid) return;
  token_num = pos.t_end;
  __nv_bfloat16* qb = reinterpret_cast<__nv_bfloat16*>(smem_co + CO_QB);
  __nv_bfloat16* kb = reinterpret_cast<__nv_bfloat16*>(smem_co + CO_KB);
  __nv_bfloat16* sh = reinterpret_cast<__nv_bfloat16*>(smem_co + CO_SH);
  __nv_bfloat16* sl = reinterpret_cast<__nv_bfloat16*>(smem_co + CO_SL);
  __nv_bfloat16* dh = reinterpret_cast<__nv_bfloat16*>(smem_co + CO_DH);
  __nv_bfloat16* dl = reinterpret_cast<__nv_bfloat16*>(smem_co + CO_DL);
  __nv_bfloat16* ah_t = reinterpret_cast<__nv_bfloat16*>(smem_co + CO_AH);
  __nv_bfloat16* al_t = reinterpret_cast<__nv_bfloat16*>(smem_co + CO_AL);
  float* gs = reinterpret_cast<float*>(smem_co + CO_SC);  // G
  float* es = gs + CHUNK;                                 // exp(G)
  const int chunk = pos.chunk, h = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int t0 = pos.t0;
  const int64_t ch = static_cast<int64_t>(chunk) * heads + h;

  // the fp32 operands (incoming state, delta) go to registers first: their latency hides behind the q/k staging and
  // the q k^T product, and they are split into bf16 pairs afterwards
  constexpr int S_PER_THREAD = GDN_D * GDN_D / 4 / GC_THREADS, D_PER_THREAD = CHUNK * GDN_D / 4 / GC_THREADS;
  float4 s_regs[S_PER_THREAD], d_regs[D_PER_THREAD];
  {
    const float4* s_src = reinterpret_cast<const float4*>(chunk_state + ch * GDN_D * GDN_D);
    const float4* d_src = reinterpret_cast<const float4*>(delta + ch * CHUNK * GDN_D);
#pragma unroll
    for (int j = 0; j < S_PER_THREAD; ++j) s_regs[j] = s_src[tid + j * GC_THREADS];
#pragma unroll
    for (int j = 0; j < D_PER_THREAD; ++j) d_regs[j] = d_src[tid + j * GC_THREADS];
  }
  load_rows_bf16(qb, q + h * q_h, q_t, t0, token_num, tid);
  load_rows_bf16(kb, k + h * k_h, k_t, t0, token_num, tid);
  if (tid < CHUNK) {
    gs[tid] = g_cumsum[ch * CHUNK + tid];
    es[tid] = expf(gs[tid]);
  }
  __syncthreads();
  const int mt = warp & 3, nh = warp >> 2, gr = lane >> 2, tg = (lane & 3) * 2;
  // ---- att[t][i] = <q_t, k_i> exp(G_t - G_i) for i <= t, both tokens valid; kept as a bf16 pair (left operand of
  //      att @ delta)
  {
    float acc[4][4];
    causal_scores(acc, qb, kb, mt, nh, lane);
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int t = mt * 16 + gr + half * 8, i = nh * 32 + nt * 8 + tg;
        const bool row_ok = t0 + t < token_num;
        const float a0 = (row_ok && i <= t) ? acc[nt][2 * half] * expf(gs[t] - gs[i]) : 0.f;
        const float a1 = (row_ok && i + 1 <= t) ? acc[nt][2 * half + 1] * expf(gs[t] - gs[i + 1]) : 0.f;
        uint32_t hi, lo;
        split_pair(a0, a1, hi, lo);
        *reinterpret_cast<uint32_t*>(ah_t + t * GC_P64 + i) = hi;
        *reinterpret_cast<uint32_t*>(al_t + t * GC_P64 + i) = lo;
      }
  }
  {
    auto stage = [&](const float4& x, __nv_bfloat16* hi, __nv_bfloat16* lo, int i) {  // i = float4 index in [rows][128]
      uint32_t h0, l0, h1, l1;
      split_pair(x.x, x.y, h0, l0);
      split_pair(x.z, x.w, h1, l1);
      *reinterpret_cast<uint2*>(hi + (i >> 5) * GC_P128 + (i & 31) * 4) = make_uint2(h0, h1);
      *reinterpret_cast<uint2*>(lo + (i >> 5) * GC_P128 + (i & 31) * 4) = make_uint2(l0, l1);
    };
#pragma unroll
    for (int j = 0; j < S_PER_THREAD; ++j) stage(s_regs[j], sh, sl, tid + j * GC_THREADS);
#pragma unroll
    for (int j = 0; j < D_PER_THREAD; ++j) stage(d_regs[j], dh, dl, tid + j * GC_THREADS);
  }
  __syncthreads();
  // ---- out = exp(G) (q @ S_in) + att @ delta: warp = (16-row tile mt, 64-column half nh)
  float acc[8][4];
#pragma unroll
  for (int nt = 0; nt < 8; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
#pragma unroll 2
  for (int ks = 0; ks < GDN_D / 16; ++ks) {
    uint32_t a[4];
    frag_a(a, qb, GC_P128, mt * 16, ks * 16, lane);
#pragma unroll
    for (int np = 0; np < 4; ++np) {
      uint32_t bh[4], bl[4];
      frag_b_kn(bh, sh, GC_P128, ks * 16, nh * 64 + np * 16, lane);
      frag_b_kn(bl, sl, GC_P128, ks * 16, nh * 64 + np * 16, lane);
      mma_bf16_16816(acc[2 * np], a, bh[0], bh[1]);
      mma_bf16_16816(acc[2 * np], a, bl[0], bl[1]);
      mma_bf16_16816(acc[2 * np + 1], a, bh[2], bh[3]);
      mma_bf16_16816(acc[2 * np + 1], a, bl[2], bl[3]);
    }
  }
  {
    const float e0 = es[mt * 16 + gr], e1 = es[mt * 16 + gr + 8];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      acc[nt][0] *= e0;
      acc[nt][1] *= e0;
      acc[nt][2] *= e1;
      acc[nt][3] *= e1;
    }
  }
  for (int ks = 0; ks <= mt; ++ks) {  // att is lower triangular
    uint32_t ah[4], al[4];
    frag_a(ah, ah_t, GC_P64, mt * 16, ks * 16, lane);
    frag_a(al, al_t, GC_P64, mt * 16, ks * 16, lane);
#pragma unroll
    for (int np = 0; np < 4; ++np) {
      uint32_t bh[4], bl[4];
      frag_b_kn(bh, dh, GC_P128, ks * 16, nh * 64 + np * 16, lane);
      frag_b_kn(bl, dl, GC_P128, ks * 16, nh * 64 + np * 16, lane);
      mma_bf16_16816(acc[2 * np], ah, bh[0], bh[1]);
      mma_bf16_16816(acc[2 * np], ah, bl[0], bl[1]);
      mma_bf16_16816(acc[2 * np], al, bh[0], bh[1]);
      mma_bf16_16816(acc[2 * np + 1], ah, bh[2], bh[3]);
      mma_bf16_16816(acc[2 * np + 1], ah, bl[2], bl[3]);
      mma_bf16_16816(acc[2 * np + 1], al, bh[2], bh[3]);
    }
  }
#pragma unroll
  for (int nt = 0; nt < 8; ++nt)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int64_t t = t0 + mt * 16 + gr + half * 8;
      if (t < token_num)
        *reinterpret_cast<uint32_t*>(out + t * o_t + h * o_h + nh * 64 + nt * 8 + tg) =
            pack_bf16(acc[nt][2 * half], acc[nt][2 * half + 1]);
    }
}

template <typename K>
static int set_smem(K kernel, int bytes, bool* flag_per_device, const char* what) {
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !flag_per_device[dev]) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess)
      return fail(ERR_RUNTIME, "%s: cannot raise dynamic shared memory to %d", what, bytes);
    // two CTAs of the prepare and state kernels fit one SM only with the largest shared-memory carveout (a hint)
    cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
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
