// Gated-DeltaNet chunk-64 prefill over a packed batch as ONE kernel on the 5th-generation tensor cores.
//
// One CTA walks the chunks of one (sequence, head) pair; the state never leaves the SM.  It computes what the
// reference's three operators compute together (triton_kernels/gdn_recurrent_prefill.py:248-396 prepare_wy,
// :404-537 chunk_state, :563-690 chunk_output; math in the comment block :329-342) without their HBM intermediates:
//   G = cumsum(g);  L[t,i] = beta_t e^{G_t-G_i} <k_t,k_i> (i<t);  (I+L) u = beta v;  (I+L) w = beta e^G k
//   delta = u - w S;  o_t = e^{G_t} q_t S + sum_{i<=t} <q_t,k_i> e^{G_t-G_i} delta_i;  S <- e^{G_last} S + k^T (e^{G_last-G} delta)
// Every matrix product runs as tcgen05.mma (bf16 inputs, fp32 accumulation in tensor memory) in the TRANSPOSED
// orientation, so that the 128 value columns are the MMA's M dimension and a thread that owns value column dv
// owns tensor-memory lane dv:
//   D1  [128 x 64]  = [Q;K] K^T            rows 0-63 <q_t,k_i>, rows 64-127 <k_t,k_i>   (operands exact in bf16)
//   Dd  [dv x t]    = S^T w^T              -> delta^T = u^T - Dd
//   O1  [dv x t]    = S^T q^T,   O2 [dv x t] = delta^T A^T     -> out^T = e^{G_t} O1 + O2
//   S^T [dv x dk]  += delta'^T k           (accumulated in place in tensor memory after the decay scaling)
// fp32 operands (S, w, delta, A) are fed as a bf16 pair hi + lo with the three cross products hi*hi, hi*lo, lo*hi
// (two when the other operand is exact), which keeps about 16 mantissa bits: the same order of accuracy as the
// reference's 3xTF32 products.  P = (I + L)^-1 is formed in fp32 on the CUDA cores by a blocked inverse (16 x 16 diagonal
// blocks by forward substitution, two levels of P21 = -P22 L21 P11 with register tiles); the classical
// delta = P beta (v - e^G k S) then needs P only as the right-hand operand of one tensor-core product, so w never exists.
// Q/K/V chunks arrive by tensor-map TMA (128-byte swizzle) straight from the strided [T, H, 128] activations.
#include "b200_attn.h"
#include "gdn_inverse.cuh"
#include "umma.cuh"

namespace b200 {

// warps 0-3: value columns (u, delta, out); warps 4-7: key columns (w) and the state; thread 0 also issues the TMA
// loads and the MMAs.  Eight warps = two per scheduler, so every thread may hold up to 255 registers (the solve
// keeps a 64-entry column in registers); a ninth warp would cut that to 168.
constexpr int GF_THREADS = 256;
constexpr int GF_LP = INV_LP;     // fp32 pitch of L rows: float4 rows, conflict-free for row-per-lane stores

// shared-memory map (bytes from a 1024-aligned base); every operand tile is a swizzled [rows][128 B] block set
constexpr int GF_SH = 0;                   // S^T hi [128 dv][128 dk]: 2 blocks x 16 KiB
constexpr int GF_SL = GF_SH + 32768;       // S^T lo
constexpr int GF_QK = GF_SL + 32768;       // [Q;K] stacked: block b at b*16 KiB = 64 Q rows (8 KiB) then 64 K rows
constexpr int GF_V = GF_QK + 32768;        // V [64 t][128 dv]: 2 blocks x 8 KiB
constexpr int GF_WH = GF_V + 16384;        // w^T hi [128 dk][64 t]; later delta'^T hi [128 dv][64 t]
constexpr int GF_WL = GF_WH + 16384;
constexpr int GF_DH = GF_WL + 16384;       // delta^T hi [128 dv][64 t]
constexpr int GF_DL = GF_DH + 16384;
constexpr int GF_AH = GF_DL + 16384;       // A hi [64 t][64 i]
constexpr int GF_AL = GF_AH + 8192;
constexpr int GF_L = GF_AL + 8192;         // L fp32 [64][GF_LP]
constexpr int GF_SC = GF_L + CHUNK * GF_LP * 4;  // per-token scalars, 4 arrays of 64 floats
constexpr int GF_SMEM = GF_SC + 4 * CHUNK * 4 + 1024;
static_assert(GF_SMEM <= 227 * 1024, "shared memory budget");

// tensor-memory columns
constexpr uint32_t TM_D1 = 0, TM_DD = 64, TM_O1 = 128, TM_M = 192, TM_O2 = 256, TM_S = 320, TM_COLS = 512;  // O1|M adjacent

struct GdnFusedParams {
  const float* beta;
  const float* g;
  const int32_t* cu_seqlens;
  float* state;
  __nv_bfloat16* out;
  int* err;
  int64_t be_t, be_h, g_t, g_h, o_t, o_h;
  int heads;
};

__device__ __forceinline__ void split8(const float (&v)[8], uint4& hi, uint4& lo) {
  uint32_t h[4], l[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const __nv_bfloat16 h0 = __float2bfloat16_rn(v[2 * j]), h1 = __float2bfloat16_rn(v[2 * j + 1]);
    const float r0 = v[2 * j] - __bfloat162float(h0), r1 = v[2 * j + 1] - __bfloat162float(h1);
    h[j] = static_cast<uint32_t>(__bfloat16_as_ushort(h0)) | (static_cast<uint32_t>(__bfloat16_as_ushort(h1)) << 16);
    l[j] = pack_bf16(r0, r1);
  }
  hi = make_uint4(h[0], h[1], h[2], h[3]);
  lo = make_uint4(l[0], l[1], l[2], l[3]);
}

__global__ void __launch_bounds__(GF_THREADS, 1)
gdn_chunk_fused_kernel(const __grid_constant__ GdnFusedParams p, const __grid_constant__ CUtensorMap map_q,
                       const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ uint64_t bar_load, bar_mma, bar_aux;
  __shared__ uint32_t tmem_slot;
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* Lm = reinterpret_cast<float*>(smem + GF_L);
  float* s_beta = reinterpret_cast<float*>(smem + GF_SC);  // beta_t (0 for padding)
  float* s_G = s_beta + CHUNK;                             // G_t
  float* s_eG = s_G + CHUNK;                               // e^{G_t}
  float* s_dec = s_eG + CHUNK;                             // e^{G_last - G_t} (0 for padding)
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int h = blockIdx.x, b = blockIdx.y;
  const int tok0 = p.cu_seqlens[b];
  const int len = p.cu_seqlens[b + 1] - tok0;
  const int num_chunks = (len + CHUNK - 1) / CHUNK;
  const bool issuer = tid == 0;

  if (warp == 0) tmem_alloc(&tmem_slot, TM_COLS);
  if (tid == 0) {
    mbar_init(&bar_load, 1);
    mbar_init(&bar_mma, 1);
    mbar_init(&bar_aux, 1);
    mbar_fence_init();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = tmem_slot;
  const uint32_t tlane = tmem + (static_cast<uint32_t>(32 * (warp & 3)) << 16);  // this warp's lane quarter
  const uint32_t sbase = smem_u32(smem);

  auto issue_loads = [&](int c) {
    const int t0 = tok0 + c * CHUNK;
    mbar_expect_tx(&bar_load, 3 * CHUNK * GDN_D * 2);
    tma_load_4d(smem + GF_QK, &map_q, 0, t0, 0, h, &bar_load);
    tma_load_4d(smem + GF_QK + 8192, &map_k, 0, t0, 0, h, &bar_load);
    tma_load_4d(smem + GF_QK + 16384, &map_q, 0, t0, 1, h, &bar_load);
    tma_load_4d(smem + GF_QK + 24576, &map_k, 0, t0, 1, h, &bar_load);
    tma_load_4d(smem + GF_V, &map_v, 0, t0, 0, h, &bar_load);
  };
  // g and beta of tokens lane and lane+32 of a chunk (warp 0 only); fetched one chunk ahead
  float g0 = 0.f, g1 = 0.f, b0 = 0.f, b1 = 0.f;
  auto fetch_scalars = [&](int c) {
    const int t0 = tok0 + c * CHUNK, valid = min(CHUNK, len - c * CHUNK);
    const bool ok0 = lane < valid, ok1 = lane + 32 < valid;
    g0 = ok0 ? p.g[static_cast<int64_t>(t0 + lane) * p.g_t + h * p.g_h] : 0.f;
    g1 = ok1 ? p.g[static_cast<int64_t>(t0 + lane + 32) * p.g_t + h * p.g_h] : 0.f;
    b0 = ok0 ? p.beta[static_cast<int64_t>(t0 + lane) * p.be_t + h * p.be_h] : 0.f;
    b1 = ok1 ? p.beta[static_cast<int64_t>(t0 + lane + 32) * p.be_t + h * p.be_h] : 0.f;
  };
  if (num_chunks > 0) {
    if (issuer) issue_loads(0);
    if (warp == 0) fetch_scalars(0);
  }

  uint32_t mma_phase = 0, aux_phase = 0;
  bool failed = false;
  for (int c = 0; c < num_chunks; ++c) {
    const int t0 = tok0 + c * CHUNK;
    const int valid = min(CHUNK, len - c * CHUNK);
    const bool last = c + 1 == num_chunks;
    // ---- per-token scalars: warp 0 scans g (tokens lane and lane+32)
    if (warp == 0) {
      const bool ok0 = lane < valid, ok1 = lane + 32 < valid;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float a = __shfl_up_sync(0xffffffffu, g0, o), bb = __shfl_up_sync(0xffffffffu, g1, o);
        if (lane >= o) {
          g0 += a;
          g1 += bb;
        }
      }
      g1 += __shfl_sync(0xffffffffu, g0, 31);
      const float g_last = __shfl_sync(0xffffffffu, g1, 31);
      s_beta[lane] = b0;
      s_beta[lane + 32] = b1;
      s_G[lane] = g0;
      s_G[lane + 32] = g1;
      s_eG[lane] = expf(g0);
      s_eG[lane + 32] = expf(g1);
      s_dec[lane] = ok0 ? expf(g_last - g0) : 0.f;
      s_dec[lane + 32] = ok1 ? expf(g_last - g1) : 0.f;
    }
    // ---- Q, K, V of this chunk
    bool ok = mbar_wait_bounded(&bar_load, c & 1);
    if (__syncthreads_or(!ok)) { failed = true; break; }
    // ---- D1 = [Q;K] K^T
    if (issuer) {
      tc_fence_after_sync();
      const uint32_t idesc = idesc_bf16_f32(128, 64, false, false);
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        const uint32_t a = sbase + GF_QK + (ks >> 2) * 16384 + (ks & 3) * 32;
        umma_ss(tmem + TM_D1, smem_desc_sw128(a, 16, 1024), smem_desc_sw128(a + 8192, 16, 1024), idesc, ks > 0);
      }
      umma_commit(&bar_mma);
    }
    ok = mbar_wait_bounded(&bar_mma, mma_phase & 1);
    ++mma_phase;
    if (__syncthreads_or(!ok)) { failed = true; break; }
    tc_fence_after_sync();
    // ---- D1 -> A (bf16 pair, B operand of the output product) and L (fp32, for the inverse)
    {
      const int half = warp >> 2, r = 32 * (warp & 3) + lane;
      constexpr float LOG2E = 1.4426950408889634f;
      uint32_t d[32];
      tmem_ld32(tlane + TM_D1 + half * 32, d);
      tmem_ld_wait();
      if (r < CHUNK) {
        const int t = r;
        const float gt = s_G[t];
        const bool row_ok = t < valid;
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
          float a8[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int i = half * 32 + cc * 8 + j;
            a8[j] = (row_ok && i <= t) ? ex2_fast((gt - s_G[i]) * LOG2E) * __uint_as_float(d[cc * 8 + j]) : 0.f;
          }
          uint4 hi, lo;
          split8(a8, hi, lo);
          const uint32_t off = t * 128 + (((half * 4 + cc) ^ (t & 7)) << 4);
          *reinterpret_cast<uint4*>(smem + GF_AH + off) = hi;
          *reinterpret_cast<uint4*>(smem + GF_AL + off) = lo;
        }
        fence_proxy_async();
      } else {
        const int t = r - CHUNK;
        const float gt = s_G[t], bt = s_beta[t];  // beta is 0 on padding rows
#pragma unroll
        for (int cc = 0; cc < 8; ++cc) {
          float l4[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int i = half * 32 + cc * 4 + j;
            l4[j] = (i < t) ? bt * ex2_fast((gt - s_G[i]) * LOG2E) * __uint_as_float(d[cc * 4 + j]) : 0.f;
          }
          *reinterpret_cast<float4*>(Lm + t * GF_LP + half * 32 + cc * 4) = make_float4(l4[0], l4[1], l4[2], l4[3]);
        }
      }
    }
    tc_fence_before_sync();
    __syncthreads();
    // ---- warps 0-3: P = (I + L)^-1 in fp32 on the CUDA cores, blocked: the four 16x16 diagonal blocks by forward
    //      substitution (one thread per column), then two levels of  P21 = -P22 (L21 P11)  with 4x4 register tiles;
    //      then Pu[t][i] = P[t][i] beta_i as a bf16 pair (B operand of the delta product) over the dead L.
    //      warps 4-7 meanwhile: R^T[dv][i] = v_i[dv] - e^{G_i} M^T[dv][i] as a bf16 pair (A operand of the delta
    //      product) over the w tiles, then the decay of the state in tensor memory.
    if (warp < 4) {
      float* Pm = reinterpret_cast<float*>(smem + GF_DH);                      // [64][GF_LP] over the delta tiles
      float* Tm = reinterpret_cast<float*>(smem + GF_DH + CHUNK * GF_LP * 4);  // merge scratch, [32][INV_TP]
      blocked_inverse64(Lm, Pm, Tm, tid);
      named_barrier(4, 128);
      {
        const int t = tid >> 1, i0 = (tid & 1) * 32;
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
          const float4 p0 = *reinterpret_cast<const float4*>(Pm + t * GF_LP + i0 + cc * 8);
          const float4 p1 = *reinterpret_cast<const float4*>(Pm + t * GF_LP + i0 + cc * 8 + 4);
          const float pv[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
          float pu[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int i = i0 + cc * 8 + j;
            pu[j] = (i <= t) ? pv[j] * s_beta[i] : 0.f;  // blocks above the diagonal were never written
          }
          uint4 hi, lo;
          split8(pu, hi, lo);
          const uint32_t off = t * 128 + ((((i0 >> 3) + cc) ^ (t & 7)) << 4);
          *reinterpret_cast<uint4*>(smem + GF_L + off) = hi;
          *reinterpret_cast<uint4*>(smem + GF_L + 8192 + off) = lo;
        }
      }
      fence_proxy_async();
    } else {
      const int dv = tid - 128;
      if (c > 0) {
        // the two products that only need the incoming state, as one N=128 product: [O1 | M^T] = S^T [Q;K]^T
        if (tid == 128) {
          tc_fence_after_sync();
          const uint32_t idesc = idesc_bf16_f32(128, 128, false, false);
#pragma unroll
          for (int grp = 0; grp < 2; ++grp) {
            const uint32_t sa = sbase + (grp == 0 ? GF_SH : GF_SL);
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
              const uint32_t o = (ks >> 2) * 16384 + (ks & 3) * 32;
              umma_ss(tmem + TM_O1, smem_desc_sw128(sa + o, 16, 1024), smem_desc_sw128(sbase + GF_QK + o, 16, 1024),
                      idesc, (grp | ks) != 0);
            }
          }
          umma_commit(&bar_aux);
        }
        ok = mbar_wait_bounded(&bar_aux, aux_phase & 1);
        tc_fence_after_sync();
      }
      const uint8_t* vcol = smem + GF_V + (dv >> 6) * 8192 + (dv & 7) * 2;
      const int vch = (dv & 63) >> 3;
#pragma unroll 1  // rolled: the phase's code stays a half / a quarter as long (instruction cache)
      for (int hf = 0; hf < 2; ++hf) {
        uint32_t d[32];
        if (c > 0) {
          tmem_ld32(tlane + TM_M + hf * 32, d);
          tmem_ld_wait();
        }
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
          float r8[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int i = hf * 32 + cc * 8 + j;
            const uint16_t raw = *reinterpret_cast<const uint16_t*>(vcol + i * 128 + ((vch ^ (i & 7)) << 4));
            const float vv = __uint_as_float(static_cast<uint32_t>(raw) << 16);
            r8[j] = c > 0 ? fmaf(-s_eG[i], __uint_as_float(d[cc * 8 + j]), vv) : vv;
          }
          uint4 hi, lo;
          split8(r8, hi, lo);
          const uint32_t off = dv * 128 + (((hf * 4 + cc) ^ (dv & 7)) << 4);
          *reinterpret_cast<uint4*>(smem + GF_WH + off) = hi;
          *reinterpret_cast<uint4*>(smem + GF_WL + off) = lo;
        }
      }
      fence_proxy_async();
      if (c > 0) {
        const float decay = s_eG[CHUNK - 1];
        uint32_t d[32];
#pragma unroll 1  // rolled: the phase's code stays a half / a quarter as long (instruction cache)
        for (int qd = 0; qd < 4; ++qd) {
          tmem_ld32(tlane + TM_S + qd * 32, d);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) d[j] = __float_as_uint(__uint_as_float(d[j]) * decay);
          tmem_st32(tlane + TM_S + qd * 32, d);
        }
        tmem_st_wait();
      }
    }
    if (c > 0) ++aux_phase;
    tc_fence_before_sync();
    if (__syncthreads_or(!ok)) { failed = true; break; }
    // ---- delta^T = R^T Pu^T  (hi*hi + hi*lo + lo*hi)
    if (issuer) {
      tc_fence_after_sync();
      const uint32_t idesc = idesc_bf16_f32(128, 64, false, false);
#pragma unroll
      for (int grp = 0; grp < 3; ++grp) {
        const uint32_t ra = sbase + (grp == 2 ? GF_WL : GF_WH), pb = sbase + GF_L + (grp == 1 ? 8192 : 0);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          umma_ss(tmem + TM_DD, smem_desc_sw128(ra + ks * 32, 16, 1024), smem_desc_sw128(pb + ks * 32, 16, 1024), idesc,
                  (grp | ks) != 0);
      }
      umma_commit(&bar_mma);
    }
    ok = mbar_wait_bounded(&bar_mma, mma_phase & 1);
    ++mma_phase;
    if (__syncthreads_or(!ok)) { failed = true; break; }
    tc_fence_after_sync();
    // ---- delta^T -> delta (pair) and delta' = e^{G_last - G} delta (pair, over the dead R tiles); all eight warps,
    //      32 tokens each
    {
      const int dv = tid & 127, hf = warp >> 2;
      uint32_t d[32];
      tmem_ld32(tlane + TM_DD + hf * 32, d);
      tmem_ld_wait();
#pragma unroll
      for (int cc = 0; cc < 4; ++cc) {
        float v8[8], s8[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          v8[j] = __uint_as_float(d[cc * 8 + j]);
          s8[j] = v8[j] * s_dec[hf * 32 + cc * 8 + j];
        }
        uint4 hi, lo;
        const uint32_t off = dv * 128 + (((hf * 4 + cc) ^ (dv & 7)) << 4);
        split8(v8, hi, lo);
        *reinterpret_cast<uint4*>(smem + GF_DH + off) = hi;
        *reinterpret_cast<uint4*>(smem + GF_DL + off) = lo;
        split8(s8, hi, lo);
        *reinterpret_cast<uint4*>(smem + GF_WH + off) = hi;
        *reinterpret_cast<uint4*>(smem + GF_WL + off) = lo;
      }
      fence_proxy_async();
    }
    tc_fence_before_sync();
    __syncthreads();
    // ---- O2 = delta^T A^T, S^T += delta'^T k
    if (issuer) {
      tc_fence_after_sync();
      const uint32_t idesc_kk = idesc_bf16_f32(128, 64, false, false);
#pragma unroll
      for (int grp = 0; grp < 3; ++grp) {
        const uint32_t da = sbase + (grp == 1 ? GF_DL : GF_DH), ab = sbase + (grp == 2 ? GF_AL : GF_AH);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          umma_ss(tmem + TM_O2, smem_desc_sw128(da + ks * 32, 16, 1024), smem_desc_sw128(ab + ks * 32, 16, 1024),
                  idesc_kk, (grp | ks) != 0);
      }
      const uint32_t idesc_s = idesc_bf16_f32(128, 128, false, true);
#pragma unroll
      for (int grp = 0; grp < 2; ++grp) {
        const uint32_t da = sbase + (grp == 0 ? GF_WH : GF_WL);
#pragma unroll
        for (int kt = 0; kt < 4; ++kt)
          umma_ss(tmem + TM_S, smem_desc_sw128(da + kt * 32, 16, 1024),
                  smem_desc_sw128(sbase + GF_QK + 8192 + kt * 2048, 16384, 1024), idesc_s, c > 0 || (grp | kt) != 0);
      }
      umma_commit(&bar_mma);
    }
    ok = mbar_wait_bounded(&bar_mma, mma_phase & 1);
    ++mma_phase;
    if (__syncthreads_or(!ok)) { failed = true; break; }
    tc_fence_after_sync();
    if (!last) {  // every reader of Q, K and V is done
      if (issuer) issue_loads(c + 1);
      if (warp == 0) fetch_scalars(c + 1);
    }
    // ---- value threads: out^T = e^{G_t} O1 + O2;  key threads: export the state (bf16 pair for the next chunk,
    //      fp32 to global memory after the last one)
    if (warp < 4) {
      // out^T -> [t][dv] bf16 staged in the (now free) delta tile, then whole rows go out as 16-byte stores
      const int dv = tid;
      __nv_bfloat16* stage = reinterpret_cast<__nv_bfloat16*>(smem + GF_DH);
#pragma unroll 1  // rolled: the phase's code stays a half / a quarter as long (instruction cache)
      for (int hf = 0; hf < 2; ++hf) {
        uint32_t o2[32], o1[32];
        tmem_ld32(tlane + TM_O2 + hf * 32, o2);
        if (c > 0) tmem_ld32(tlane + TM_O1 + hf * 32, o1);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const int t = hf * 32 + j;
          float o = __uint_as_float(o2[j]);
          if (c > 0) o = fmaf(s_eG[t], __uint_as_float(o1[j]), o);
          stage[t * GDN_D + dv] = __float2bfloat16_rn(o);
        }
      }
      named_barrier(1, 128);
      __nv_bfloat16* obase = p.out + static_cast<int64_t>(t0) * p.o_t + h * p.o_h;
      for (int idx = tid; idx < valid * 16; idx += 128) {
        const int row = idx >> 4, c16 = idx & 15;
        *reinterpret_cast<uint4*>(obase + static_cast<int64_t>(row) * p.o_t + c16 * 8) =
            *reinterpret_cast<const uint4*>(stage + row * GDN_D + c16 * 8);
      }
    } else {
      const int dv = tid - 128;
      uint32_t d[32];
#pragma unroll 1  // rolled: the phase's code stays a half / a quarter as long (instruction cache)
      for (int qd = 0; qd < 4; ++qd) {
        tmem_ld32(tlane + TM_S + qd * 32, d);
        tmem_ld_wait();
        if (last) {
          // final state: fp32 [dk][dv] staged over the (now free) state tiles, stored by one 64 KiB bulk copy
          float* stage = reinterpret_cast<float*>(smem + GF_SH);
#pragma unroll
          for (int j = 0; j < 32; ++j) stage[(qd * 32 + j) * GDN_D + dv] = __uint_as_float(d[j]);
        } else {
#pragma unroll
          for (int cc = 0; cc < 4; ++cc) {
            float v8[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) v8[j] = __uint_as_float(d[cc * 8 + j]);
            uint4 hi, lo;
            split8(v8, hi, lo);
            const int chunk16 = qd * 4 + cc;  // 16-byte chunk along dk (0..15)
            const uint32_t off = (chunk16 >> 3) * 16384 + dv * 128 + (((chunk16 & 7) ^ (dv & 7)) << 4);
            *reinterpret_cast<uint4*>(smem + GF_SH + off) = hi;
            *reinterpret_cast<uint4*>(smem + GF_SL + off) = lo;
          }
        }
      }
      fence_proxy_async();
      if (last) {
        named_barrier(2, 128);
        if (tid == 128) {
          bulk_s2g(p.state + (static_cast<int64_t>(b) * p.heads + h) * GDN_D * GDN_D, smem + GF_SH,
                   GDN_D * GDN_D * 4);
          bulk_wait_read();
        }
      }
    }
    tc_fence_before_sync();
    __syncthreads();
  }
  if (num_chunks == 0 && warp >= 4) {  // empty sequence: zero state
    float* srow = p.state + (static_cast<int64_t>(b) * p.heads + h) * GDN_D * GDN_D + (tid - 128);
    for (int j = 0; j < GDN_D; ++j) srow[j * GDN_D] = 0.f;
  }
  if (failed && tid == 0) atomicExch(p.err, 1);
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, TM_COLS);
}

// {64 dims, T tokens, 2 column blocks, H heads} over a strided [T, H, 128] bf16 activation
static bool encode_qkv_map(CUtensorMap* map, const void* base, int64_t tokens, int64_t stride_t, int64_t stride_h,
                           int heads, uint32_t box_blocks) {
  const uint64_t dims[4] = {64, static_cast<uint64_t>(tokens), 2, static_cast<uint64_t>(heads)};
  const uint64_t strides[3] = {static_cast<uint64_t>(stride_t) * 2, 128, static_cast<uint64_t>(stride_h) * 2};
  const uint32_t box[4] = {64, CHUNK, box_blocks, 1};
  return encode_map_bf16_sw128(map, base, 4, dims, strides, box);
}

}  // namespace b200

using namespace b200;

extern "C" int b200_gdn_chunked_prefill_fused(const void* q, int64_t q_stride_t, int64_t q_stride_h, const void* k,
                                              int64_t k_stride_t, int64_t k_stride_h, const void* v,
                                              int64_t v_stride_t, int64_t v_stride_h, const float* beta,
                                              int64_t beta_stride_t, int64_t beta_stride_h, const float* g,
                                              int64_t g_stride_t, int64_t g_stride_h, const int32_t* cu_seqlens,
                                              int32_t batch, int32_t total_tokens, float* state, void* out,
                                              int64_t out_stride_t, int64_t out_stride_h, int32_t num_heads,
                                              int32_t key_dim, int32_t value_dim, b200_stream_t stream) {
  B200_REQUIRE(batch > 0 && batch <= 65535 && total_tokens > 0 && num_heads > 0 && num_heads <= 65535,
               "gdn_chunked_prefill_fused: bad shape");
  B200_REQUIRE(key_dim == GDN_D && value_dim == GDN_D, "gdn_chunked_prefill_fused: key/value dim must be %d (got %d/%d)",
               GDN_D, key_dim, value_dim);
  B200_REQUIRE(cu_seqlens != nullptr, "gdn_chunked_prefill_fused: cu_seqlens is required");
  B200_REQUIRE(aligned16(out) && aligned16(state) && out_stride_t % 8 == 0 && out_stride_h % 8 == 0,
               "gdn_chunked_prefill_fused: out and state must be 16-byte aligned, out strides multiples of 8 elements");
  B200_REQUIRE(aligned16(q) && aligned16(k) && aligned16(v) && q_stride_t % 8 == 0 && k_stride_t % 8 == 0 &&
                   v_stride_t % 8 == 0 && q_stride_h % 8 == 0 && k_stride_h % 8 == 0 && v_stride_h % 8 == 0,
               "gdn_chunked_prefill_fused: q/k/v must be 16-byte aligned with token and head strides that are "
               "multiples of 8 elements");
  CUtensorMap mq, mk, mv;
  if (!encode_qkv_map(&mq, q, total_tokens, q_stride_t, q_stride_h, num_heads, 1) ||
      !encode_qkv_map(&mk, k, total_tokens, k_stride_t, k_stride_h, num_heads, 1) ||
      !encode_qkv_map(&mv, v, total_tokens, v_stride_t, v_stride_h, num_heads, 2))
    return fail(ERR_RUNTIME, "gdn_chunked_prefill_fused: cannot encode the q/k/v tensor maps");
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    if (cudaFuncSetAttribute(gdn_chunk_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, GF_SMEM) != cudaSuccess)
      return fail(ERR_RUNTIME, "gdn_chunked_prefill_fused: cannot raise dynamic shared memory to %d", GF_SMEM);
    configured[dev] = true;
  }
  GdnFusedParams p;
  p.beta = beta;
  p.g = g;
  p.cu_seqlens = cu_seqlens;
  p.state = state;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.err = wait_timeout_flag();
  if (!p.err) return fail(ERR_RUNTIME, "gdn_chunked_prefill_fused: no error flag");
  p.be_t = beta_stride_t; p.be_h = beta_stride_h;
  p.g_t = g_stride_t; p.g_h = g_stride_h;
  p.o_t = out_stride_t; p.o_h = out_stride_h;
  p.heads = num_heads;
  gdn_chunk_fused_kernel<<<dim3(num_heads, batch), GF_THREADS, GF_SMEM, reinterpret_cast<cudaStream_t>(stream)>>>(
      p, mq, mk, mv);
  return check_launch("gdn_chunked_prefill_fused");
}
