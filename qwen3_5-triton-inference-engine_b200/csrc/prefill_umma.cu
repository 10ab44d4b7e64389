// Packed variable-length causal GQA prefill attention on the Blackwell tensor cores (tcgen05 + TMEM + tensor-map TMA).
//   b200_gqa_varlen_causal       <-> triton_kernels/gqa_attention_varlen_causal.py:214-278 (kernel :99-210)
//   b200_fused_prefill_attention <-> the chain of engine/runner.py:339-384: partial_rope(q), partial_rope(k),
//                                    gqa_attention_varlen_causal, attention_gate_pack, paged_kv_fill_varlen
//
// One CTA = one (sequence, kv head, block of 32 query tokens).  The 4 Q heads of the group are stacked into the 128
// rows of one MMA tile (row = token*4 + head, the stacking idea of gqa_attention_varlen_causal.py:151-160), so every
// K/V tile is fetched once per group.  Per 128-token KV tile:
//     S[128 x 128]  = Q[128 x 256] . K^T          tcgen05.mma, both operands K-major in shared memory, D in TMEM
//     P = exp2(S*scale*log2e - m)                  two softmax threads per row (64 columns each), TMEM -> TMEM
//     O[128 x 256] += P[128 x 128] . V[128 x 256]  tcgen05.mma, P from TMEM, V as an MN-major operand, O stays in TMEM
// The tile is 128 tokens wide because a tcgen05.mma with M=128 costs at least ~64 cycles whatever its N (measured:
// N=64 and N=128 both ~69 cycles per instruction, N=256 128 cycles), so N=64 score tiles ran the tensor pipe at half
// rate.  Roles: warps 0-7 softmax/epilogue (TMEM lane quarter = warp % 4, column half = warp / 4), warp 8 issues the
// MMAs (the whole warp walks the loop, lane 0 issues), warps 9 and 10 issue the K and V TMA loads (64 KiB per tile,
// 128-byte swizzle, no multicast; two independent chains so that K of tile j+1 is requested the moment S of tile j
// is done).  S is double-buffered in TMEM (2 x 128 columns + 256 for O = all 512) and P never touches shared memory:
// the softmax threads store it as packed bf16 over the first 64 columns of the S buffer they just read, and the PV
// product takes its A operand from tensor memory.  Q, K and V are single-buffered in shared memory.  O is rescaled in TMEM only when a row maximum grows by more than 2^8 (the
// running reference maximum may lag; p then stays <= 256, exact for bf16 and fp32 l).
// The reference's rounding points are kept where they matter for the 2e-2 bar: p is rounded to bf16 for the PV
// product while l sums the fp32 p; scores are scaled in fp32 (the reference pre-scales q and re-rounds it to bf16).
// Every mbarrier wait is bounded; on expiry the role sets the device error flag and the CTA drains and exits.
#include "b200_attn.h"
#include "umma.cuh"

namespace b200 {

constexpr int PU_BQ = 32;
constexpr int PU_TKV = 128;
constexpr int PU_SOFTMAX_THREADS = 256;
constexpr int PU_THREADS = 352;                     // 8 softmax warps + MMA issuer + K producer + V producer
constexpr int PU_Q_BYTES = 128 * HEAD_DIM * 2;      // 64 KiB: 4 column blocks of [128 rows][64]
constexpr int PU_KV_BYTES = PU_TKV * HEAD_DIM * 2;  // 64 KiB: 4 column blocks of [128 rows][64]
constexpr int PU_SMEM = PU_Q_BYTES + 2 * PU_KV_BYTES;  // 192 KiB; tiles need 1024-byte alignment: the kernel checks
constexpr int PU_OUT_PITCH = HEAD_DIM * 2 + 16;     // staging pitch of the epilogue (bytes)
static_assert(128 * PU_OUT_PITCH <= PU_Q_BYTES + PU_KV_BYTES, "output staging must fit in the Q + K region");
constexpr uint32_t PU_TMEM_COLS = 512;              // S0 [0,128) S1 [128,256) (P over their first 64) O [256,512)
constexpr float PU_TAU = 8.0f;                      // lazy-rescale threshold (log2 domain)
constexpr float PU_LOG2E = 1.4426950408889634f;

struct PrefillUmmaParams {
  int num_kv_heads, batch_wide_order;
  __nv_bfloat16* out;
  int64_t out_t, out_h;
  const int32_t* cu_seqlens;
  int* err;
  float scale_log2;
  // fused form only: rotary embedding of q in shared memory, sigmoid gate in the epilogue
  const __nv_bfloat16* gate;
  int64_t gate_t;
  const void* position_ids;
  int ids_are_int64;
  const float* inv_freq;
};

// Fused path, first kernel: rotate K at its position, scatter K (rotated) and V into the paged cache and keep a
// packed copy of the rotated K [T, H_kv, 256] for the attention kernel's TMA loads (so the rotation is computed once
// per token, not once per consumer tile).  One warp per (token, kv head) row, each lane 8 consecutive dims;
// grid = (pages of the longest sequence, H_kv, B).
__global__ void __launch_bounds__(128)
rope_scatter_kernel(const __nv_bfloat16* __restrict__ k, int64_t k_t, int64_t k_h, const __nv_bfloat16* __restrict__ v,
                    int64_t v_t, int64_t v_h, __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache,
                    int64_t kc_p, int64_t kc_h, int64_t kc_s, int64_t vc_p, int64_t vc_h, int64_t vc_s,
                    const int32_t* __restrict__ block_table, int64_t bt_b, const int32_t* __restrict__ cu_seqlens,
                    const void* __restrict__ position_ids, int ids_are_int64, const float* __restrict__ inv_freq,
                    int rotary_half, __nv_bfloat16* __restrict__ k_rot, int num_kv_heads) {
  const int lp = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  pdl_trigger();  // the attention kernel behind this one may start: it waits for this grid before it reads k_rot
  const int seq_start = cu_seqlens[b];
  const int seq_len = cu_seqlens[b + 1] - seq_start;
  if (lp * PAGE >= seq_len) return;
  const int64_t phys = block_table[b * bt_b + lp];
  const int lanes_half = rotary_half / 8;
  const bool in_rot = lane < 2 * lanes_half;
  const bool first = lane < lanes_half;
  const int partner = first ? lane + lanes_half : lane - lanes_half;
  const int dbase = (in_rot ? (first ? lane : partner) : 0) * 8;
  const float freq = lane < rotary_half ? inv_freq[lane] : 0.f;  // rotary_half <= 32: one angle per lane
  // a warp's four token rows (slots warp, warp + 4, ...): every row's loads are requested before the first is used
  constexpr int ROWS = PAGE / 4;
  uint4 kraw[ROWS], vraw[ROWS];
  int64_t pid[ROWS];
#pragma unroll
  for (int i = 0; i < ROWS; ++i) {
    const int tok = lp * PAGE + warp + 4 * i;
    if (tok < seq_len) {
      const int64_t t = seq_start + tok;
      kraw[i] = *reinterpret_cast<const uint4*>(k + t * k_t + h * k_h + lane * 8);
      vraw[i] = *reinterpret_cast<const uint4*>(v + t * v_t + h * v_h + lane * 8);
      pid[i] = rotary_half == 0 ? 0
               : ids_are_int64 ? static_cast<const int64_t*>(position_ids)[t]
                               : static_cast<int64_t>(static_cast<const int32_t*>(position_ids)[t]);
    }
  }
#pragma unroll
  for (int i = 0; i < ROWS; ++i) {
    const int slot = warp + 4 * i;
    const int tok = lp * PAGE + slot;
    if (tok >= seq_len) break;
    const int64_t t = seq_start + tok;
    uint32_t kw[4] = {kraw[i].x, kraw[i].y, kraw[i].z, kraw[i].w};
    if (rotary_half > 0) {
      // the warp computes the row's angles once, one sincosf per lane, and hands them round by shuffles (the same
      // full-range sincosf of float(pos) * inv_freq as before, so the rotated bytes do not change)
      float sn = 0.f, cs = 1.f;
      if (lane < rotary_half) sincosf(static_cast<float>(pid[i]) * freq, &sn, &cs);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t other = __shfl_sync(0xffffffffu, kw[j], in_rot ? partner : lane);
        const float s0 = __shfl_sync(0xffffffffu, sn, dbase + 2 * j), c0 = __shfl_sync(0xffffffffu, cs, dbase + 2 * j);
        const float s1 = __shfl_sync(0xffffffffu, sn, dbase + 2 * j + 1), c1 = __shfl_sync(0xffffffffu, cs, dbase + 2 * j + 1);
        if (in_rot) {
          const uint32_t fa = first ? kw[j] : other;
          const uint32_t fb = first ? other : kw[j];
          float f0, g0, f1, g1;
          rope_pair(bf16_lo(fa), bf16_lo(fb), s0, c0, f0, g0);
          rope_pair(bf16_hi(fa), bf16_hi(fb), s1, c1, f1, g1);
          kw[j] = first ? pack_bf16(f0, f1) : pack_bf16(g0, g1);
        }
      }
    }
    const uint4 krot = make_uint4(kw[0], kw[1], kw[2], kw[3]);
    *reinterpret_cast<uint4*>(k_cache + phys * kc_p + h * kc_h + slot * kc_s + lane * 8) = krot;
    *reinterpret_cast<uint4*>(k_rot + (t * num_kv_heads + h) * HEAD_DIM + lane * 8) = krot;
    *reinterpret_cast<uint4*>(v_cache + phys * vc_p + h * vc_h + slot * vc_s + lane * 8) = vraw[i];
  }
}



template <bool FUSED>
__global__ void __launch_bounds__(PU_THREADS, 1)
varlen_causal_umma_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                          const __grid_constant__ CUtensorMap map_v, const __grid_constant__ PrefillUmmaParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ uint64_t bar_q, bar_qr, bar_k, bar_v, bar_s[2], bar_p[2], bar_pv;
  __shared__ uint32_t tmem_slot;
  __shared__ float xm[2][2][128];  // [tile parity][column half][row]: row maxima (at the end: row sums) exchanged
                                   // between the two threads of a row

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // Two block orders (blocks are scheduled x-fastest).  Batch-wide: grid = (sequences x kv heads, query blocks), so the
  // whole batch's last (heaviest) query blocks run first, then the ones before them, ... and the one-tile blocks at
  // the start of every sequence fill the tail: longest-processing-time-first over the launch.  Taken when the K/V of
  // the whole batch fits the L2 several times over.  Per sequence: grid = (query blocks, kv heads, sequences), heaviest
  // block of a sequence first; the CTAs that run together then share one or two sequences' K/V tiles in the L2.
  const bool batch_wide = p.batch_wide_order != 0;
  const int qb = batch_wide ? gridDim.y - 1 - blockIdx.y : gridDim.x - 1 - blockIdx.x;
  const int h = batch_wide ? blockIdx.x % p.num_kv_heads : blockIdx.y;
  const int b = batch_wide ? blockIdx.x / p.num_kv_heads : blockIdx.z;
  const int seq_start = p.cu_seqlens[b];
  const int seq_len = p.cu_seqlens[b + 1] - seq_start;
  const int q0 = qb * PU_BQ;
  if (q0 >= seq_len) {
    if (FUSED) pdl_wait();  // every CTA orders the grid after the kernel in front of it
    return;
  }
  const int kv_end = min(q0 + PU_BQ, seq_len);
  const int n_tiles = (kv_end + PU_TKV - 1) / PU_TKV;

  uint8_t* smem = smem_raw;
  if ((smem_u32(smem) & 1023u) != 0) {  // swizzled tiles need 1024-byte alignment; never taken with __align__(1024)
    if (tid == 0) atomicExch(p.err, 1);
    return;
  }
  uint8_t* q_s = smem;
  uint8_t* k_s = smem + PU_Q_BYTES;
  uint8_t* v_s = k_s + PU_KV_BYTES;

  if (warp == 0) tmem_alloc(&tmem_slot, PU_TMEM_COLS);
  if (tid == 0) {
    mbar_init(&bar_q, 1);
    mbar_init(&bar_qr, 128);
    mbar_init(&bar_k, 1);
    mbar_init(&bar_v, 1);
    mbar_init(&bar_s[0], 1);
    mbar_init(&bar_s[1], 1);
    mbar_init(&bar_p[0], PU_SOFTMAX_THREADS);  // one per S/P buffer: a warp may be a tile ahead of another
    mbar_init(&bar_p[1], PU_SOFTMAX_THREADS);
    mbar_init(&bar_pv, 1);
    mbar_fence_init();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = tmem_slot;
  const uint32_t tmem_o = tmem + 2 * PU_TKV;

  if (warp == 9) {
    // ------------------------------------------------------------------ TMA producer: Q once, then the K tiles
    if (lane == 0) {
      bool ok = true;
      mbar_expect_tx(&bar_q, PU_Q_BYTES);
      tma_load_5d(q_s, &map_q, 0, 0, h, seq_start + q0, 0, &bar_q);
      // fused form: started while the rope + scatter kernel still runs (programmatic dependent launch).  Everything up
      // to here - tensor-memory allocation, barriers, the Q tile, and the V tiles of the other producer - overlaps with
      // it; the rotated K it writes is read only after it has completed.
      if (FUSED) pdl_wait();
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (j >= 1) ok = mbar_wait_bounded(&bar_s[(j - 1) & 1], ((j - 1) >> 1) & 1);  // S of tile j-1 done: K free
        if (!ok) break;
        mbar_expect_tx(&bar_k, PU_KV_BYTES);
        tma_load_4d(k_s, &map_k, 0, seq_start + j * PU_TKV, 0, h, &bar_k);
      }
      if (!ok) atomicExch(p.err, 1);
    }
  } else if (warp == 10) {
    // ------------------------------------------------------------------ TMA producer: the V tiles
    if (lane == 0) {
      bool ok = true;
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (j >= 1) ok = mbar_wait_bounded(&bar_pv, (j - 1) & 1);  // PV of tile j-1 done: V free
        if (!ok) break;
        mbar_expect_tx(&bar_v, PU_KV_BYTES);
        tma_load_4d(v_s, &map_v, 0, seq_start + j * PU_TKV, 0, h, &bar_v);
      }
      if (!ok) atomicExch(p.err, 1);
    }
  } else if (warp == 8) {
    // ------------------------------------------------------------------ MMA issuer
    {
      // the whole warp walks the loop (uniform control flow), lane 0 issues
      const bool leader = lane == 0;
      const uint32_t idesc_s = idesc_bf16_f32(128, PU_TKV, false, false);
      const uint32_t idesc_o = idesc_bf16_f32(128, HEAD_DIM, false, true);
      const uint32_t q_addr = smem_u32(q_s), k_addr = smem_u32(k_s), v_addr = smem_u32(v_s);
      bool ok = FUSED ? mbar_wait_bounded(&bar_qr, 0) : mbar_wait_bounded(&bar_q, 0);
      auto issue_pv = [&](int jj) {
        ok = ok && mbar_wait_bounded(&bar_p[jj & 1], (jj >> 1) & 1);
        ok = ok && mbar_wait_bounded(&bar_v, jj & 1);
        if (!ok) return;
        tc_fence_after_sync();
#pragma unroll
        for (int kt = 0; kt < PU_TKV / 16; ++kt)
          umma_ts_leader(tmem_o, tmem + (jj & 1) * PU_TKV + kt * 8,  // P: 16 tokens = 8 packed columns per step
                         smem_desc_sw128(v_addr + kt * 2048, PU_TKV * 128, 1024), idesc_o, (jj > 0) || (kt > 0), leader);
        umma_commit_leader(&bar_pv, leader);
      };
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int s = j & 1;
        ok = mbar_wait_bounded(&bar_k, j & 1);
        // S(j) overwrites the buffer whose first columns hold P(j-2): the PV product that reads them from tensor
        // memory must have COMPLETED, issue order alone does not protect an operand in tensor memory
        if (ok && j >= 2) ok = mbar_wait_bounded(&bar_pv, (j - 2) & 1);
        if (!ok) break;
        tc_fence_after_sync();
#pragma unroll
        for (int ks = 0; ks < HEAD_DIM / 16; ++ks) {
          const uint32_t o = (ks >> 2) * (128 * 128) + (ks & 3) * 32;
          umma_ss_leader(tmem + s * PU_TKV, smem_desc_sw128(q_addr + o, 16, 1024), smem_desc_sw128(k_addr + o, 16, 1024),
                         idesc_s, ks > 0, leader);
        }
        umma_commit_leader(&bar_s[s], leader);
        if (j >= 1) issue_pv(j - 1);
      }
      if (ok) issue_pv(n_tiles - 1);
      if (!ok && leader) atomicExch(p.err, 1);
    }
  } else {
    // ------------------------------------------------------------------ softmax + epilogue
    const int row = 32 * (warp & 3) + lane;    // TMEM lane; row = token*4 + head
    const int half = warp >> 2;                // this thread's 64 of the tile's 128 columns
    const int q_tok = q0 + (row >> 2);
    const uint32_t lane_base = static_cast<uint32_t>(32 * (warp & 3)) << 16;
    const int pair_bar = 1 + (warp & 3);       // named barrier of the two warps that share these rows
    float m_ref = -INFINITY, l_run = 0.f;
    bool ok = true;
    if (FUSED && half == 0) {
      // rotary embedding of this row's q in place (dims [0,32) and [32,64) live in column block 0, chunks c, c+4)
      const int64_t t = seq_start + min(q_tok, seq_len - 1);
      const int64_t pid = p.ids_are_int64 ? static_cast<const int64_t*>(p.position_ids)[t]
                                          : static_cast<int64_t>(static_cast<const int32_t*>(p.position_ids)[t]);
      const float posf = static_cast<float>(pid);
      // the four rows of a token share their angles: each lane of a quad computes 8 of the 32 (sin, cos) pairs
      float sn[8], cs[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) sincosf(posf * p.inv_freq[(lane & 3) * 8 + i], &sn[i], &cs[i]);
      ok = mbar_wait_bounded(&bar_q, 0);
      uint8_t* qrow = q_s + row * 128;
#pragma unroll
      for (int c = 0; c < 4; ++c) {  // chunk c holds dims [8c, 8c+8), chunk c+4 their partners [32+8c, 40+8c)
        uint4* pa = reinterpret_cast<uint4*>(qrow + ((c ^ (row & 7)) << 4));
        uint4* pb = reinterpret_cast<uint4*>(qrow + (((c + 4) ^ (row & 7)) << 4));
        const uint4 va = *pa, vb = *pb;
        uint32_t wa[4] = {va.x, va.y, va.z, va.w}, wb[4] = {vb.x, vb.y, vb.z, vb.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          // angle index 8c + 2k (+1) lives in lane (quad base + c), register 2k (+1)
          const int src = (lane & ~3) + c;
          const float c0 = __shfl_sync(0xffffffffu, cs[2 * k], src), s0 = __shfl_sync(0xffffffffu, sn[2 * k], src);
          const float c1 = __shfl_sync(0xffffffffu, cs[2 * k + 1], src), s1 = __shfl_sync(0xffffffffu, sn[2 * k + 1], src);
          float f0, g0, f1, g1;
          rope_pair(bf16_lo(wa[k]), bf16_lo(wb[k]), s0, c0, f0, g0);
          rope_pair(bf16_hi(wa[k]), bf16_hi(wb[k]), s1, c1, f1, g1);
          wa[k] = pack_bf16(f0, f1);
          wb[k] = pack_bf16(g0, g1);
        }
        *pa = make_uint4(wa[0], wa[1], wa[2], wa[3]);
        *pb = make_uint4(wb[0], wb[1], wb[2], wb[3]);
      }
      fence_proxy_async();  // the rotated rows must be visible to the tensor core's reads
      mbar_arrive(&bar_qr);
    }
    // A failed (timed-out) wait clears `ok`; the loop then keeps only its barriers and arrivals, so that the partner
    // warp and the MMA issuer are never left waiting for this thread.
    for (int j = 0; j < n_tiles; ++j) {
      const int s = j & 1;
      if (ok) ok = mbar_wait_bounded(&bar_s[s], (j >> 1) & 1);
      uint32_t r0[32], r1[32];
      float m_half = 0.f;
      if (ok) {
        tc_fence_after_sync();
        tmem_ld32(tmem + lane_base + s * PU_TKV + half * 64, r0);
        tmem_ld32(tmem + lane_base + s * PU_TKV + half * 64 + 32, r1);
        tmem_ld_wait();
        // mask (causal and inside the sequence; only tiles on the diagonal or at the sequence end need it) and take
        // the row maximum of the raw scores; the scale (> 0) is folded into the exponent below
        const int lim = min(q_tok, seq_len - 1) - j * PU_TKV - half * 64;  // last valid column of this half
        if (lim < 63) {
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            if (c > lim) r0[c] = 0xff800000u;       // -inf
            if (c + 32 > lim) r1[c] = 0xff800000u;
          }
        }
        float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
        for (int c = 0; c < 32; c += 2) {
          mx0 = fmaxf(mx0, __uint_as_float(r0[c]));
          mx1 = fmaxf(mx1, __uint_as_float(r0[c + 1]));
          mx2 = fmaxf(mx2, __uint_as_float(r1[c]));
          mx3 = fmaxf(mx3, __uint_as_float(r1[c + 1]));
        }
        m_half = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
      }
      xm[s][half][row] = m_half;
      named_barrier(pair_bar, 64);
      // after this barrier both threads of the row hold their scores in registers: the S buffer may take P
      if (ok) {
        const float m_tile = fmaxf(m_half, xm[s][half ^ 1][row]) * p.scale_log2;
        const float m_new = fmaxf(m_ref, m_tile);  // both threads of a row compute the same value
        if (j == 0) {
          m_ref = m_new;
        } else {
          const bool need = (m_new - m_ref) > PU_TAU;
          if (__any_sync(__activemask(), need)) {
            // O must be at rest before it is rescaled: wait for the PV product of tile j-1
            ok = mbar_wait_bounded(&bar_pv, (j - 1) & 1);
            tc_fence_after_sync();
            const float alpha = need ? ex2_fast(m_ref - m_new) : 1.f;
#pragma unroll 1
            for (int c0 = 0; c0 < HEAD_DIM / 2; c0 += 32) {  // this thread's 128 columns of O
              uint32_t o[32];
              tmem_ld32(tmem_o + lane_base + half * (HEAD_DIM / 2) + c0, o);
              tmem_ld_wait();
#pragma unroll
              for (int c = 0; c < 32; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * alpha);
              tmem_st32(tmem_o + lane_base + half * (HEAD_DIM / 2) + c0, o);
            }
            tmem_st_wait();
            l_run *= alpha;
            if (need) m_ref = m_new;
          }
        }
        // p = 2^(s*scale - m_ref): fp32 for l, bf16 for the PV product, stored as this thread's 32 packed columns of
        // the P tile (tokens 2c, 2c+1 in column c) over the S buffer
        float sum0 = 0.f, sum1 = 0.f;
        const float neg_m = -m_ref, sc = p.scale_log2;
        uint32_t w[32];
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          const float x0 = ex2_fast(fmaf(__uint_as_float(c < 16 ? r0[2 * c] : r1[2 * c - 32]), sc, neg_m));
          const float x1 = ex2_fast(fmaf(__uint_as_float(c < 16 ? r0[2 * c + 1] : r1[2 * c - 31]), sc, neg_m));
          sum0 += x0;
          sum1 += x1;
          w[c] = pack_bf16(x0, x1);
        }
        l_run += sum0 + sum1;
        tmem_st32(tmem + lane_base + s * PU_TKV + half * 32, w);
        tmem_st_wait();
      }
      tc_fence_before_sync();   // this thread's TMEM loads/stores before the arrive
      mbar_arrive(&bar_p[s]);
    }
    // ---- epilogue: O / l -> bf16 -> staged in shared memory (Q and K are dead) -> coalesced global stores
    // A parity wait only tells the two most recent phases apart, and this thread may not have seen the PV product of
    // tile n-2 complete yet: wait for it first, then for the last one.
    if (ok && n_tiles >= 2) ok = mbar_wait_bounded(&bar_pv, (n_tiles - 2) & 1);
    if (ok) ok = mbar_wait_bounded(&bar_pv, (n_tiles - 1) & 1);
    float* xl = &xm[n_tiles & 1][0][0];  // the parity slot the last tile did not use
    xl[half * 128 + row] = l_run;
    named_barrier(pair_bar, 64);
    if (ok) {
      tc_fence_after_sync();
      const float inv_l = 1.f / (l_run + xl[(half ^ 1) * 128 + row]);
      uint8_t* orow = smem + row * PU_OUT_PITCH + half * HEAD_DIM;  // this half's 128 columns = 256 bytes
#pragma unroll 1
      for (int c0 = 0; c0 < HEAD_DIM / 2; c0 += 32) {
        uint32_t o[32];
        tmem_ld32(tmem_o + lane_base + half * (HEAD_DIM / 2) + c0, o);
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
    named_barrier(9, PU_SOFTMAX_THREADS);  // the eight softmax warps only
    if (ok) {
      // 128 rows x 32 sixteen-byte chunks; a warp covers one 512-byte row per step.  The gate rows are fetched
      // eight steps at a time so that their latency is paid once per batch, not once per chunk.
      constexpr int STEPS = 128 * (HEAD_DIM / 8) / PU_SOFTMAX_THREADS;  // 16 iterations of 256 threads
#pragma unroll 1
      for (int i0 = 0; i0 < STEPS; i0 += 8) {
        uint4 gv[8];
        if (FUSED) {
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const int i = (i0 + u) * PU_SOFTMAX_THREADS + tid, r = i >> 5, ch = i & 31;
            const int tok = min(q0 + (r >> 2), seq_len - 1);
            gv[u] = *reinterpret_cast<const uint4*>(p.gate + static_cast<int64_t>(seq_start + tok) * p.gate_t +
                                                    (h * GROUP + (r & 3)) * HEAD_DIM + ch * 8);
          }
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int i = (i0 + u) * PU_SOFTMAX_THREADS + tid, r = i >> 5, ch = i & 31;
          const int tok = q0 + (r >> 2);
          if (tok < seq_len) {
            uint4 v = *reinterpret_cast<const uint4*>(smem + r * PU_OUT_PITCH + ch * 16);
            if (FUSED) {
              uint32_t xs[4] = {v.x, v.y, v.z, v.w};
              const uint32_t gs[4] = {gv[u].x, gv[u].y, gv[u].z, gv[u].w};
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                xs[k] = pack_bf16(bf16_lo(xs[k]) * sigmoid_fast(bf16_lo(gs[k])),
                                  bf16_hi(xs[k]) * sigmoid_fast(bf16_hi(gs[k])));
              }
              v = make_uint4(xs[0], xs[1], xs[2], xs[3]);
            }
            *reinterpret_cast<uint4*>(p.out + static_cast<int64_t>(seq_start + tok) * p.out_t +
                                      (h * GROUP + (r & 3)) * p.out_h + ch * 8) = v;
          }
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

// Encodes the tensor maps and launches the attention kernel (FUSED adds rope on q and the output gate).
template <bool FUSED>
static int launch_prefill_umma(const void* q, int64_t q_stride_t, int64_t q_stride_h, const void* k, int64_t k_stride_t,
                               int64_t k_stride_h, const void* v, int64_t v_stride_t, int64_t v_stride_h,
                               PrefillUmmaParams p, int batch, int total_tokens, int max_seqlen, int num_kv_heads,
                               cudaStream_t stream, const char* what) {
  CUtensorMap map_q, map_k, map_v;
  const uint64_t T = static_cast<uint64_t>(total_tokens), H = static_cast<uint64_t>(num_kv_heads);
  {
    // q as {64 cols, 4 heads of a group, groups, tokens, 4 column blocks}; one load = 32 tokens of one group
    const uint64_t dims[5] = {64, GROUP, H, T, HEAD_DIM / 64};
    const uint64_t strides[4] = {static_cast<uint64_t>(q_stride_h) * 2, static_cast<uint64_t>(q_stride_h) * 2 * GROUP,
                                 static_cast<uint64_t>(q_stride_t) * 2, 128};
    const uint32_t box[5] = {64, GROUP, 1, PU_BQ, HEAD_DIM / 64};
    if (!encode_map_bf16_sw128(&map_q, q, 5, dims, strides, box))
      return fail(ERR_RUNTIME, "%s: cannot encode the tensor map of q", what);
  }
  {
    // k, v as {64 cols, tokens, 4 column blocks, kv heads}; one load = 64 tokens of one head
    const uint64_t dims[4] = {64, T, HEAD_DIM / 64, H};
    const uint32_t box[4] = {64, PU_TKV, HEAD_DIM / 64, 1};
    const uint64_t ks[3] = {static_cast<uint64_t>(k_stride_t) * 2, 128, static_cast<uint64_t>(k_stride_h) * 2};
    const uint64_t vs[3] = {static_cast<uint64_t>(v_stride_t) * 2, 128, static_cast<uint64_t>(v_stride_h) * 2};
    if (!encode_map_bf16_sw128(&map_k, k, 4, dims, ks, box) || !encode_map_bf16_sw128(&map_v, v, 4, dims, vs, box))
      return fail(ERR_RUNTIME, "%s: cannot encode the tensor maps of k / v", what);
  }
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    if (cudaFuncSetAttribute(varlen_causal_umma_kernel<FUSED>, cudaFuncAttributeMaxDynamicSharedMemorySize, PU_SMEM) !=
        cudaSuccess)
      return fail(ERR_RUNTIME, "%s: cannot raise dynamic shared memory to %d", what, PU_SMEM);
    configured[dev] = true;
  }
  p.err = wait_timeout_flag();
  if (!p.err) return fail(ERR_RUNTIME, "%s: no error flag", what);
  p.scale_log2 = (1.0f / sqrtf(static_cast<float>(HEAD_DIM))) * PU_LOG2E;
  B200_REQUIRE((max_seqlen + PU_BQ - 1) / PU_BQ <= 65535 && batch <= 65535 && num_kv_heads <= 65535,
               "%s: max_seqlen must be at most %d, batch and heads at most 65535 (got %d, %d, %d)", what, 65535 * PU_BQ,
               max_seqlen, batch, num_kv_heads);
  const int q_blocks = (max_seqlen + PU_BQ - 1) / PU_BQ;
  // K and V of the batch (bf16): below a quarter of the 126 MB L2 every running CTA finds its tiles there whatever the order
  p.batch_wide_order = static_cast<int64_t>(total_tokens) * num_kv_heads * HEAD_DIM * 4 <= (32ll << 20) ? 1 : 0;
  p.num_kv_heads = num_kv_heads;
  const dim3 grid = p.batch_wide_order ? dim3(static_cast<unsigned>(num_kv_heads) * batch, q_blocks, 1)
                                       : dim3(q_blocks, num_kv_heads, batch);
  // the fused form starts behind its own rope + scatter kernel while that one still runs (see the K producer)
  if (launch_pdl(FUSED, varlen_causal_umma_kernel<FUSED>, grid, dim3(PU_THREADS), PU_SMEM, stream, map_q, map_k, map_v, p) !=
      cudaSuccess)
    return fail(ERR_LAUNCH, "%s: %s", what, cudaGetErrorString(cudaGetLastError()));
  return check_launch(what);
}

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
  PrefillUmmaParams p = {};
  p.out = static_cast<__nv_bfloat16*>(out);
  p.out_t = out_stride_t;
  p.out_h = out_stride_h;
  p.cu_seqlens = cu_seqlens;
  return launch_prefill_umma<false>(q, q_stride_t, q_stride_h, k, k_stride_t, k_stride_h, v, v_stride_t, v_stride_h, p,
                                    batch, total_tokens, max_seqlen, num_kv_heads,
                                    reinterpret_cast<cudaStream_t>(stream), "gqa_varlen_causal");
}

extern "C" int b200_fused_prefill_attention(const void* q, int64_t q_stride_t, int64_t q_stride_h, const void* k,
                                            int64_t k_stride_t, int64_t k_stride_h, const void* v, int64_t v_stride_t,
                                            int64_t v_stride_h, const void* gate, int64_t gate_stride_t, void* k_cache,
                                            void* v_cache, int64_t kc_stride_p, int64_t kc_stride_h,
                                            int64_t kc_stride_s, int64_t vc_stride_p, int64_t vc_stride_h,
                                            int64_t vc_stride_s, const int32_t* block_table, int64_t bt_stride_b,
                                            const int32_t* cu_seqlens, const void* position_ids, int32_t ids_are_int64,
                                            const float* inv_freq, int32_t rotary_dim, void* k_rot_scratch, void* out,
                                            int32_t batch, int32_t total_tokens, int32_t max_seqlen,
                                            int32_t num_q_heads, int32_t num_kv_heads, int32_t head_dim,
                                            b200_stream_t stream) {
  B200_REQUIRE(batch > 0 && batch <= 65535, "fused_prefill_attention: batch must be in [1, 65535]");
  B200_REQUIRE(total_tokens > 0, "fused_prefill_attention: total_tokens must be positive");
  B200_REQUIRE(head_dim == HEAD_DIM, "fused_prefill_attention: head_dim must be %d (got %d)", HEAD_DIM, head_dim);
  B200_REQUIRE(num_kv_heads > 0 && num_q_heads == num_kv_heads * GROUP,
               "fused_prefill_attention: needs %d Q heads per KV head (got %d/%d)", GROUP, num_q_heads, num_kv_heads);
  B200_REQUIRE(rotary_dim == 64, "fused_prefill_attention: rotary_dim must be 64 (got %d)", rotary_dim);
  B200_REQUIRE(inv_freq != nullptr && position_ids != nullptr && k_rot_scratch != nullptr,
               "fused_prefill_attention: NULL rope inputs or scratch");
  B200_REQUIRE(aligned16(q) && aligned16(k) && aligned16(v) && aligned16(out) && aligned16(gate) &&
                   aligned16(k_cache) && aligned16(v_cache) && aligned16(k_rot_scratch) && mult8(q_stride_t) &&
                   mult8(q_stride_h) && mult8(k_stride_t) && mult8(k_stride_h) && mult8(v_stride_t) &&
                   mult8(v_stride_h) && mult8(gate_stride_t) && mult8(kc_stride_p) && mult8(kc_stride_h) &&
                   mult8(kc_stride_s) && mult8(vc_stride_p) && mult8(vc_stride_h) && mult8(vc_stride_s),
               "fused_prefill_attention: tensors must be 16-byte aligned with strides that are multiples of 8");
  if (max_seqlen <= 0) return OK;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const dim3 grid((max_seqlen + PAGE - 1) / PAGE, num_kv_heads, batch);
  rope_scatter_kernel<<<grid, 128, 0, st>>>(
      static_cast<const __nv_bfloat16*>(k), k_stride_t, k_stride_h, static_cast<const __nv_bfloat16*>(v), v_stride_t,
      v_stride_h, static_cast<__nv_bfloat16*>(k_cache), static_cast<__nv_bfloat16*>(v_cache), kc_stride_p, kc_stride_h,
      kc_stride_s, vc_stride_p, vc_stride_h, vc_stride_s, block_table, bt_stride_b, cu_seqlens, position_ids,
      ids_are_int64, inv_freq, rotary_dim / 2, static_cast<__nv_bfloat16*>(k_rot_scratch), num_kv_heads);
  int rc = check_launch("fused_prefill_attention (rope + scatter)");
  if (rc != OK) return rc;
  PrefillUmmaParams p = {};
  p.out = static_cast<__nv_bfloat16*>(out);
  p.out_t = static_cast<int64_t>(num_q_heads) * HEAD_DIM;
  p.out_h = HEAD_DIM;
  p.cu_seqlens = cu_seqlens;
  p.gate = static_cast<const __nv_bfloat16*>(gate);
  p.gate_t = gate_stride_t;
  p.position_ids = position_ids;
  p.ids_are_int64 = ids_are_int64;
  p.inv_freq = inv_freq;
  return launch_prefill_umma<true>(q, q_stride_t, q_stride_h, k_rot_scratch, static_cast<int64_t>(num_kv_heads) * HEAD_DIM,
                                   HEAD_DIM, v, v_stride_t, v_stride_h, p, batch, total_tokens, max_seqlen,
                                   num_kv_heads, st, "fused_prefill_attention");
}
