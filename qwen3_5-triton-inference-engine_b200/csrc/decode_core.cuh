// Warp-level core of paged GQA decode attention (4 Q heads per KV head, head_dim 256, 16-token pages).
//
// One warp owns one stream of KV pages.  Pages are staged in shared memory by the TMA engine
// (cp.async.bulk, one 512-byte copy per token row so rows can sit at a 528-byte pitch: ldmatrix then
// reads eight rows from eight different bank groups).  Scores use tokens as the MMA M dimension:
//   S^T[16 tok x 8]   = K_page[16 x 256] . Q^T[256 x 8]      (Q heads 4..7 are zero padding)
//   O^T[256 x 8]     += V_page^T[256 x 16] . P^T[16 x 8]
// so the 4-head group costs an N=8 tile instead of an M=16 one.  Softmax statistics live in registers and
// are reduced over tokens with warp shuffles.  Arithmetic follows the reference kernel
// (triton_kernels/gqa_attention_decode_paged.py:699-721): fp32 scores times scale, p = exp(s - m) in fp32,
// p rounded to bf16 for the PV product while l accumulates the unrounded p.
#pragma once
#include "common.cuh"

namespace b200 {

constexpr int ROW_BYTES = HEAD_DIM * 2;          // 512: one token row of K or V
constexpr int ROW_PITCH = ROW_BYTES + 16;        // 528: padded pitch in shared memory
constexpr int TILE_BYTES = PAGE * ROW_PITCH;     // 8448: one staged K (or V) page
constexpr int STAGE_BYTES = 2 * TILE_BYTES;      // K tile then V tile
constexpr uint32_t PAGE_TX_BYTES = 2 * PAGE * ROW_BYTES;  // bytes the mbarrier expects per stage

struct DecodeWarpState {
  uint32_t qb[16][2];  // B fragments of Q^T, one pair per 16-wide slice of head_dim
  float o[16][4];      // O^T accumulators: tile i = dims [16i,16i+16), cols = heads (lane&3)*2,+1
  float m[2], l[2];    // running max / sum for heads (lane&3)*2 and +1
};

__device__ __forceinline__ void decode_state_init(DecodeWarpState& st) {
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    st.o[i][0] = st.o[i][1] = st.o[i][2] = st.o[i][3] = 0.f;
  }
  st.m[0] = st.m[1] = -INFINITY;
  st.l[0] = st.l[1] = 0.f;
}

// Q fragments from a [4][256] bf16 tile (row pitch `pitch` elements) in global or shared memory.
__device__ __forceinline__ void decode_load_q(DecodeWarpState& st, const __nv_bfloat16* q4, int64_t pitch, int lane) {
  const int n = lane >> 2, kk = (lane & 3) * 2;
#pragma unroll
  for (int ks = 0; ks < 16; ++ks) {
    if (n < GROUP) {
      const __nv_bfloat16* row = q4 + n * pitch + ks * 16 + kk;
      st.qb[ks][0] = *reinterpret_cast<const uint32_t*>(row);
      st.qb[ks][1] = *reinterpret_cast<const uint32_t*>(row + 8);
    } else {
      st.qb[ks][0] = st.qb[ks][1] = 0u;
    }
  }
}

// Issue the copies of one page (K rows by lanes 0..15, V rows by lanes 16..31) into `stage`.
__device__ __forceinline__ void decode_issue_page(uint8_t* stage, uint64_t* bar, const __nv_bfloat16* k_page,
                                                  const __nv_bfloat16* v_page, int64_t kc_s, int64_t vc_s, int lane) {
  if (lane == 0) mbar_expect_tx(bar, PAGE_TX_BYTES);
  __syncwarp();
  const int r = lane & 15;
  if (lane < 16) {
    bulk_g2s(stage + r * ROW_PITCH, k_page + r * kc_s, ROW_BYTES, bar);
  } else {
    bulk_g2s(stage + TILE_BYTES + r * ROW_PITCH, v_page + r * vc_s, ROW_BYTES, bar);
  }
}

// Consume one staged page.  `valid` = number of leading token rows that belong to the sequence (1..16).
__device__ __forceinline__ void decode_consume_page(DecodeWarpState& st, uint8_t* stage, int valid, float scale,
                                                    int lane) {
  const uint32_t kbase = smem_u32(stage);
  const uint32_t vbase = kbase + TILE_BYTES;
  if (valid < PAGE) {
    // rows past the sequence end may hold anything (even NaN bit patterns): clear them in V so that
    // 0 * garbage cannot poison the accumulators; K garbage is removed by the -inf mask below.
    for (int i = lane; i < (PAGE - valid) * (ROW_BYTES / 16); i += 32) {
      const int r = valid + i / (ROW_BYTES / 16), c = i % (ROW_BYTES / 16);
      *reinterpret_cast<uint4*>(stage + TILE_BYTES + r * ROW_PITCH + c * 16) = make_uint4(0, 0, 0, 0);
    }
    __syncwarp();
  }
  // ---- S^T = K . Q^T
  float s[4] = {0.f, 0.f, 0.f, 0.f};
  {
    const int mi = lane >> 3, r = lane & 7;
    const uint32_t a_addr = kbase + (r + (mi & 1) * 8) * ROW_PITCH + (mi >> 1) * 16;
#pragma unroll
    for (int ks = 0; ks < 16; ++ks) {
      uint32_t a[4];
      ldmatrix_x4(a, a_addr + ks * 32);
      mma_bf16_16816(s, a, st.qb[ks][0], st.qb[ks][1]);
    }
  }
  const int tok = lane >> 2;
  s[0] = (tok < valid) ? s[0] * scale : -INFINITY;
  s[1] = (tok < valid) ? s[1] * scale : -INFINITY;
  s[2] = (tok + 8 < valid) ? s[2] * scale : -INFINITY;
  s[3] = (tok + 8 < valid) ? s[3] * scale : -INFINITY;
  // ---- online softmax over the 16 tokens (tokens live on lane>>2 and on the two row halves)
  float mx0 = fmaxf(s[0], s[2]), mx1 = fmaxf(s[1], s[3]);
#pragma unroll
  for (int o = 4; o <= 16; o <<= 1) {
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, o));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, o));
  }
  const float m0 = fmaxf(st.m[0], mx0), m1 = fmaxf(st.m[1], mx1);
  const float alpha0 = __expf(st.m[0] - m0), alpha1 = __expf(st.m[1] - m1);
  const float p0 = __expf(s[0] - m0), p1 = __expf(s[1] - m1), p2 = __expf(s[2] - m0), p3 = __expf(s[3] - m1);
  float sum0 = p0 + p2, sum1 = p1 + p3;
#pragma unroll
  for (int o = 4; o <= 16; o <<= 1) {
    sum0 += __shfl_xor_sync(0xffffffffu, sum0, o);
    sum1 += __shfl_xor_sync(0xffffffffu, sum1, o);
  }
  st.l[0] = st.l[0] * alpha0 + sum0;
  st.l[1] = st.l[1] * alpha1 + sum1;
  st.m[0] = m0;
  st.m[1] = m1;
  // P^T as the B operand: transpose the two 8x8 bf16 score fragments across the warp
  const uint32_t b0 = movmatrix_trans(pack_bf16(p0, p1));
  const uint32_t b1 = movmatrix_trans(pack_bf16(p2, p3));
  // ---- O^T = alpha * O^T + V^T . P^T
  {
    const int mi = lane >> 3, r = lane & 7;
    const uint32_t a_addr = vbase + (r + (mi >> 1) * 8) * ROW_PITCH + (mi & 1) * 16;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      uint32_t a[4];
      ldmatrix_x4_trans(a, a_addr + i * 32);
      st.o[i][0] *= alpha0;
      st.o[i][1] *= alpha1;
      st.o[i][2] *= alpha0;
      st.o[i][3] *= alpha1;
      mma_bf16_16816(st.o[i], a, b0, b1);
    }
  }
}

// Spill the warp's O^T accumulators as a row-major fp32 [4 heads][256] tile into shared memory
// (`tile` must have room for 4 KiB and be 16-byte aligned).  Lanes with (lane&3) >= 2 hold padding heads.
__device__ __forceinline__ void decode_store_acc_smem(const DecodeWarpState& st, float* tile, int lane) {
  const int h0 = (lane & 3) * 2, dr = lane >> 2;
  if (h0 < GROUP) {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      tile[h0 * HEAD_DIM + i * 16 + dr] = st.o[i][0];
      tile[(h0 + 1) * HEAD_DIM + i * 16 + dr] = st.o[i][1];
      tile[h0 * HEAD_DIM + i * 16 + 8 + dr] = st.o[i][2];
      tile[(h0 + 1) * HEAD_DIM + i * 16 + 8 + dr] = st.o[i][3];
    }
  }
}

}  // namespace b200
