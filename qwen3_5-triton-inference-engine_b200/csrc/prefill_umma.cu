// Packed variable-length causal GQA prefill attention on the Blackwell tensor cores (tcgen05 + TMEM + tensor-map TMA).
//   b200_gqa_varlen_causal <-> triton_kernels/gqa_attention_varlen_causal.py:214-278 (kernel :99-210)
//
// One CTA = one (sequence, kv head, block of 32 query tokens).  The 4 Q heads of the group are stacked into the 128
// rows of one MMA tile (row = token*4 + head, the stacking idea of gqa_attention_varlen_causal.py:151-160), so every
// K/V tile is fetched once per group.  Per 64-token KV tile:
//     S[128 x 64]   = Q[128 x 256] . K^T          tcgen05.mma, both operands K-major in shared memory, D in TMEM
//     P = exp2(S*scale*log2e - m)                  one softmax thread per row, straight out of TMEM
//     O[128 x 256] += P[128 x 64] . V[64 x 256]    tcgen05.mma, V as an MN-major operand, O stays in TMEM
// Roles: warps 0-3 softmax/epilogue (thread = row = TMEM lane), warp 4 issues the MMAs, warp 5 the TMA loads
// (Q once, K/V double-buffered, 32 KiB per copy, 128-byte swizzle, no multicast).  S is double-buffered in TMEM so
// that S of tile j+1 is computed while tile j is in the softmax.  O is rescaled in TMEM only when a row maximum
// grows by more than 2^8 (the running reference maximum may lag; p then stays <= 256, exact for bf16 and fp32 l).
// The reference's rounding points are kept where they matter for the 2e-2 bar: p is rounded to bf16 for the PV
// product while l sums the fp32 p; scores are scaled in fp32 (the reference pre-scales q and re-rounds it to bf16).
// Every mbarrier wait is bounded; on expiry the role sets the device error flag and the CTA drains and exits.
#include "b200_attn.h"
#include "umma.cuh"

namespace b200 {

constexpr int PU_BQ = 32;
constexpr int PU_TKV = 64;
constexpr int PU_THREADS = 192;
constexpr int PU_Q_BYTES = 128 * HEAD_DIM * 2;      // 64 KiB: 4 column blocks of [128 rows][64]
constexpr int PU_P_BYTES = 128 * PU_TKV * 2;        // 16 KiB: [128 rows][64]
constexpr int PU_KV_BYTES = PU_TKV * HEAD_DIM * 2;  // 32 KiB: 4 column blocks of [64 rows][64]
constexpr int PU_SMEM = PU_Q_BYTES + PU_P_BYTES + 4 * PU_KV_BYTES + 1024;
constexpr int PU_OUT_PITCH = HEAD_DIM * 2 + 16;     // staging pitch of the epilogue (bytes)
static_assert(128 * PU_OUT_PITCH <= PU_Q_BYTES + PU_P_BYTES, "output staging must fit in the Q + P region");
constexpr uint32_t PU_TMEM_COLS = 512;              // S0 [0,64) S1 [64,128) O [128,384)
constexpr float PU_TAU = 8.0f;                      // lazy-rescale threshold (log2 domain)
constexpr float PU_LOG2E = 1.4426950408889634f;

struct PrefillUmmaParams {
  __nv_bfloat16* out;
  int64_t out_t, out_h;
  const int32_t* cu_seqlens;
  int* err;
  float scale_log2;
};

__global__ void __launch_bounds__(PU_THREADS, 1)
varlen_causal_umma_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                          const __grid_constant__ CUtensorMap map_v, const __grid_constant__ PrefillUmmaParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ uint64_t bar_q, bar_k[2], bar_v[2], bar_s[2], bar_p[2], bar_pv[2];
  __shared__ uint32_t tmem_slot;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int qb = gridDim.x - 1 - blockIdx.x;  // heaviest blocks first
  const int h = blockIdx.y, b = blockIdx.z;
  const int seq_start = p.cu_seqlens[b];
  const int seq_len = p.cu_seqlens[b + 1] - seq_start;
  const int q0 = qb * PU_BQ;
  if (q0 >= seq_len) return;
  const int kv_end = min(q0 + PU_BQ, seq_len);
  const int n_tiles = (kv_end + PU_TKV - 1) / PU_TKV;

  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_s = smem;
  uint8_t* p_s = smem + PU_Q_BYTES;
  uint8_t* k_s = p_s + PU_P_BYTES;      // two stages
  uint8_t* v_s = k_s + 2 * PU_KV_BYTES;  // two stages

  if (warp == 0) tmem_alloc(&tmem_slot, PU_TMEM_COLS);
  if (tid == 0) {
    mbar_init(&bar_q, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bar_k[i], 1);
      mbar_init(&bar_v[i], 1);
      mbar_init(&bar_s[i], 1);
      mbar_init(&bar_p[i], 128);
      mbar_init(&bar_pv[i], 1);
    }
    mbar_fence_init();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = tmem_slot;
  const uint32_t tmem_o = tmem + 128;

  if (warp == 5) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      bool ok = true;
      mbar_expect_tx(&bar_q, PU_Q_BYTES);
      tma_load_5d(q_s, &map_q, 0, 0, h, seq_start + q0, 0, &bar_q);
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int s = j & 1, u = j >> 1;
        if (j >= 2) ok = mbar_wait_bounded(&bar_s[s], (u - 1) & 1);  // S of tile j-2 done: K stage free
        if (!ok) break;
        mbar_expect_tx(&bar_k[s], PU_KV_BYTES);
        tma_load_4d(k_s + s * PU_KV_BYTES, &map_k, 0, seq_start + j * PU_TKV, 0, h, &bar_k[s]);
        if (j >= 2) ok = mbar_wait_bounded(&bar_pv[s], (u - 1) & 1);  // PV of tile j-2 done: V stage free
        if (!ok) break;
        mbar_expect_tx(&bar_v[s], PU_KV_BYTES);
        tma_load_4d(v_s + s * PU_KV_BYTES, &map_v, 0, seq_start + j * PU_TKV, 0, h, &bar_v[s]);
      }
      if (!ok) atomicExch(p.err, 1);
    }
  } else if (warp == 4) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc_s = idesc_bf16_f32(128, PU_TKV, false, false);
      const uint32_t idesc_o = idesc_bf16_f32(128, HEAD_DIM, false, true);
      const uint32_t q_addr = smem_u32(q_s), p_addr = smem_u32(p_s);
      bool ok = mbar_wait_bounded(&bar_q, 0);
      auto issue_pv = [&](int jj) {
        const int s = jj & 1;
        ok = ok && mbar_wait_bounded(&bar_p[s], (jj >> 1) & 1);
        ok = ok && mbar_wait_bounded(&bar_v[s], (jj >> 1) & 1);
        if (!ok) return;
        tc_fence_after_sync();
        const uint32_t v_addr = smem_u32(v_s + s * PU_KV_BYTES);
#pragma unroll
        for (int kt = 0; kt < PU_TKV / 16; ++kt)
          umma_ss(tmem_o, smem_desc_sw128(p_addr + kt * 32, 16, 1024),
                  smem_desc_sw128(v_addr + kt * 2048, PU_TKV * 128, 1024), idesc_o, (jj > 0) || (kt > 0));
        umma_commit(&bar_pv[s]);
      };
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int s = j & 1;
        ok = mbar_wait_bounded(&bar_k[s], (j >> 1) & 1);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t k_addr = smem_u32(k_s + s * PU_KV_BYTES);
#pragma unroll
        for (int ks = 0; ks < HEAD_DIM / 16; ++ks)
          umma_ss(tmem + s * PU_TKV, smem_desc_sw128(q_addr + (ks >> 2) * (128 * 128) + (ks & 3) * 32, 16, 1024),
                  smem_desc_sw128(k_addr + (ks >> 2) * (PU_TKV * 128) + (ks & 3) * 32, 16, 1024), idesc_s, ks > 0);
        umma_commit(&bar_s[s]);
        if (j >= 1) issue_pv(j - 1);
      }
      if (ok) issue_pv(n_tiles - 1);
      if (!ok) atomicExch(p.err, 1);
    }
  } else {
    // ------------------------------------------------------------------ softmax + epilogue, thread = row
    const int row = tid;                       // TMEM lane; row = token*4 + head
    const int q_tok = q0 + (row >> 2);
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
    float m_ref = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int s = j & 1;
      ok = mbar_wait_bounded(&bar_s[s], (j >> 1) & 1);
      if (!ok) break;
      tc_fence_after_sync();
      uint32_t r0[32], r1[32];
      tmem_ld32(tmem + lane_base + s * PU_TKV, r0);
      tmem_ld32(tmem + lane_base + s * PU_TKV + 32, r1);
      tmem_ld_wait();
      // scale to the log2 domain, mask (causal and inside the sequence), row maximum
      const int lim = min(q_tok, seq_len - 1) - j * PU_TKV;  // last valid column of this tile for this row
      float m_tile = -INFINITY;
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        float a = __uint_as_float(r0[c]) * p.scale_log2, bb = __uint_as_float(r1[c]) * p.scale_log2;
        a = (c <= lim) ? a : -INFINITY;
        bb = (c + 32 <= lim) ? bb : -INFINITY;
        r0[c] = __float_as_uint(a);
        r1[c] = __float_as_uint(bb);
        m_tile = fmaxf(m_tile, fmaxf(a, bb));
      }
      const float m_new = fmaxf(m_ref, m_tile);
      if (j == 0) {
        m_ref = m_new;
      } else {
        // the P buffer is still being read by PV of tile j-1, and O must be at rest before it is rescaled
        ok = mbar_wait_bounded(&bar_pv[(j - 1) & 1], ((j - 1) >> 1) & 1);
        if (!ok) break;
        tc_fence_after_sync();
        const bool need = (m_new - m_ref) > PU_TAU;
        if (__any_sync(0xffffffffu, need)) {
          const float alpha = need ? exp2f(m_ref - m_new) : 1.f;
#pragma unroll 1
          for (int c0 = 0; c0 < HEAD_DIM; c0 += 32) {
            uint32_t o[32];
            tmem_ld32(tmem_o + lane_base + c0, o);
            tmem_ld_wait();
#pragma unroll
            for (int c = 0; c < 32; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * alpha);
            tmem_st32(tmem_o + lane_base + c0, o);
          }
          tmem_st_wait();
          l_run *= alpha;
          if (need) m_ref = m_new;
        }
      }
      // p = exp2(s - m_ref): fp32 for l, bf16 for the PV product, written as row `row` of the swizzled P tile
      float sum = 0.f;
      uint8_t* prow = p_s + row * 128;
#pragma unroll
      for (int ch = 0; ch < 8; ++ch) {
        uint32_t w[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int c = ch * 8 + k * 2;
          const float x0 = exp2f(__uint_as_float(c < 32 ? r0[c] : r1[c - 32]) - m_ref);
          const float x1 = exp2f(__uint_as_float(c + 1 < 32 ? r0[c + 1] : r1[c + 1 - 32]) - m_ref);
          sum += x0 + x1;
          w[k] = pack_bf16(x0, x1);
        }
        *reinterpret_cast<uint4*>(prow + ((ch ^ (row & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
      }
      l_run += sum;
      fence_proxy_async();      // generic-proxy stores to P before the tensor core (async proxy) reads them
      tc_fence_before_sync();   // this thread's TMEM loads/stores before the arrive
      mbar_arrive(&bar_p[s]);
    }
    // ---- epilogue: O / l -> bf16 -> staged in shared memory (Q and P are dead) -> coalesced global stores
    if (ok) ok = mbar_wait_bounded(&bar_pv[(n_tiles - 1) & 1], ((n_tiles - 1) >> 1) & 1);
    if (ok) {
      tc_fence_after_sync();
      const float inv_l = 1.f / l_run;
      uint8_t* orow = smem + row * PU_OUT_PITCH;
#pragma unroll 1
      for (int c0 = 0; c0 < HEAD_DIM; c0 += 32) {
        uint32_t o[32];
        tmem_ld32(tmem_o + lane_base + c0, o);
        tmem_ld_wait();
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint32_t w[4];
#pragma unroll
          for (int k = 0; k < 4; ++k)
            w[k] = pack_bf16(__uint_as_float(o[g * 8 + k * 2]) * inv_l, __uint_as_float(o[g * 8 + k * 2 + 1]) * inv_l);
          *reinterpret_cast<uint4*>(orow + (c0 + g * 8) * 2) = make_uint4(w[0], w[1], w[2], w[3]);
        }
      }
    } else {
      atomicExch(p.err, 1);
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");  // the four softmax warps only
    if (ok) {
      for (int i = tid; i < 128 * (HEAD_DIM / 8); i += 128) {
        const int r = i >> 5, ch = i & 31;
        const int tok = q0 + (r >> 2);
        if (tok < seq_len) {
          const uint4 v = *reinterpret_cast<const uint4*>(smem + r * PU_OUT_PITCH + ch * 16);
          *reinterpret_cast<uint4*>(p.out + static_cast<int64_t>(seq_start + tok) * p.out_t +
                                    (h * GROUP + (r & 3)) * p.out_h + ch * 8) = v;
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, PU_TMEM_COLS);
}

}  // namespace b200

using namespace b200;

static bool mult8(int64_t x) { return (x & 7) == 0; }

extern "C" int b200_gqa_varlen_causal(const void* q, int64_t q_stride_t, int64_t q_stride_h, const void* k,
                                      int64_t k_stride_t, int64_t k_stride_h, const void* v, int64_t v_stride_t,
                                      int64_t v_stride_h, void* out, int64_t out_stride_t, int64_t out_stride_h,
                                      const int32_t* cu_seqlens, int32_t batch, int32_t total_tokens,
                                      int32_t max_seqlen, int32_t num_q_heads, int32_t num_kv_heads, int32_t head_dim,
                                      b200_stream_t stream) {
  B200_REQUIRE(batch > 0 && batch <= 65535, "gqa_varlen_causal: batch must be in [1, 65535]");
  B200_REQUIRE(total_tokens > 0, "gqa_varlen_causal: total_tokens must be positive");
  B200_REQUIRE(head_dim == HEAD_DIM, "gqa_varlen_causal: head_dim must be %d (got %d)", HEAD_DIM, head_dim);
  B200_REQUIRE(num_kv_heads > 0 && num_q_heads == num_kv_heads * GROUP,
               "gqa_varlen_causal: needs %d Q heads per KV head (got %d/%d)", GROUP, num_q_heads, num_kv_heads);
  B200_REQUIRE(aligned16(q) && aligned16(k) && aligned16(v) && aligned16(out) && mult8(q_stride_t) &&
                   mult8(q_stride_h) && mult8(k_stride_t) && mult8(k_stride_h) && mult8(v_stride_t) &&
                   mult8(v_stride_h) && mult8(out_stride_t) && mult8(out_stride_h),
               "gqa_varlen_causal: tensors must be 16-byte aligned with strides that are multiples of 8");
  if (max_seqlen <= 0) return OK;
  CUtensorMap map_q, map_k, map_v;
  const uint64_t T = static_cast<uint64_t>(total_tokens), H = static_cast<uint64_t>(num_kv_heads);
  {
    // q as {64 cols, 4 heads of a group, groups, tokens, 4 column blocks}; one load = 32 tokens of one group
    const uint64_t dims[5] = {64, GROUP, H, T, HEAD_DIM / 64};
    const uint64_t strides[4] = {static_cast<uint64_t>(q_stride_h) * 2, static_cast<uint64_t>(q_stride_h) * 2 * GROUP,
                                 static_cast<uint64_t>(q_stride_t) * 2, 128};
    const uint32_t box[5] = {64, GROUP, 1, PU_BQ, HEAD_DIM / 64};
    if (!encode_map_bf16_sw128(&map_q, q, 5, dims, strides, box))
      return fail(ERR_RUNTIME, "gqa_varlen_causal: cannot encode the tensor map of q");
  }
  {
    // k, v as {64 cols, tokens, 4 column blocks, kv heads}; one load = 64 tokens of one head
    const uint64_t dims[4] = {64, T, HEAD_DIM / 64, H};
    const uint32_t box[4] = {64, PU_TKV, HEAD_DIM / 64, 1};
    const uint64_t ks[3] = {static_cast<uint64_t>(k_stride_t) * 2, 128, static_cast<uint64_t>(k_stride_h) * 2};
    const uint64_t vs[3] = {static_cast<uint64_t>(v_stride_t) * 2, 128, static_cast<uint64_t>(v_stride_h) * 2};
    if (!encode_map_bf16_sw128(&map_k, k, 4, dims, ks, box) || !encode_map_bf16_sw128(&map_v, v, 4, dims, vs, box))
      return fail(ERR_RUNTIME, "gqa_varlen_causal: cannot encode the tensor maps of k / v");
  }
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    if (cudaFuncSetAttribute(varlen_causal_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PU_SMEM) !=
        cudaSuccess)
      return fail(ERR_RUNTIME, "gqa_varlen_causal: cannot raise dynamic shared memory to %d", PU_SMEM);
    configured[dev] = true;
  }
  PrefillUmmaParams p;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.out_t = out_stride_t;
  p.out_h = out_stride_h;
  p.cu_seqlens = cu_seqlens;
  p.err = wait_timeout_flag();
  if (!p.err) return fail(ERR_RUNTIME, "gqa_varlen_causal: no error flag");
  p.scale_log2 = (1.0f / sqrtf(static_cast<float>(head_dim))) * PU_LOG2E;
  const dim3 grid((max_seqlen + PU_BQ - 1) / PU_BQ, num_kv_heads, batch);
  varlen_causal_umma_kernel<<<grid, PU_THREADS, PU_SMEM, reinterpret_cast<cudaStream_t>(stream)>>>(map_q, map_k, map_v, p);
  return check_launch("gqa_varlen_causal");
}
