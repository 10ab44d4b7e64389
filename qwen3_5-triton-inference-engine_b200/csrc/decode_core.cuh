// Warp-level core of paged GQA decode attention (4 Q heads per KV head, head_dim 256, 16-token pages).
//
// One warp owns one stream of KV pages.  A page's K tile and V tile are staged separately in shared memory by
// the TMA engine, each completing on its own mbarrier, so the score computation of a page starts as soon as its K
// rows have landed.  Two staging layouts (tile_offset<SW>): one tensor-map box per tile with the 128-byte swizzle
// (the fused kernel; dense caches), or one 512-byte bulk copy per token row at a 528-byte pitch (the drop-in split
// kernel; any cache strides); both are conflict-free for ldmatrix.  Scores use tokens as the MMA M dimension:
//   S^T[16 tok x 8]   = K_page[16 x 256] . Q^T[256 x 8]      (Q heads 4..7 are zero padding)
//   O^T[256 x 8]     += V_page^T[256 x 16] . P^T[16 x 8]
// so the 4-head group costs an N=8 tile instead of an M=16 one.  Softmax statistics live in registers; only the
// running max is reduced across lanes per page, the row sums stay per-lane partials until a state is exported.
// Arithmetic follows the reference kernel (triton_kernels/gqa_attention_decode_paged.py:699-721): fp32 scores
// times scale, p = exp(s - m) in fp32, p rounded to bf16 for the PV product while l accumulates the unrounded p.
#pragma once
#include "common.cuh"

namespace b200 {

constexpr int ROW_BYTES = HEAD_DIM * 2;                // 512: one token row of K or V
constexpr int ROW_PITCH = ROW_BYTES + 16;              // 528: padded pitch of the row-copy layout
constexpr int TILE_BYTES = PAGE * ROW_PITCH;           // 8448: one staged K (or V) tile, row-copy layout
constexpr int TILE_BYTES_SW = PAGE * ROW_BYTES;        // 8192: one staged tile, swizzled tensor-map layout
constexpr uint32_t TILE_TX_BYTES = PAGE * ROW_BYTES;   // bytes an mbarrier expects per tile

// Two shared-memory layouts of a [16 tokens][256 dims] bf16 tile:
//   SW = false  rows copied one by one (cp.async.bulk, 512 B each) to a 528-byte pitch; any cache strides.
//   SW = true   ONE tensor-map TMA box {64 dims, 16 rows, 4 column blocks} with the 128-byte swizzle: the tile is
//               4 blocks of [16 rows][128 B], 16-byte chunk c of row r stored at position c ^ (r & 7); needs a
//               dense cache and a 1024-byte aligned tile.  Both are conflict-free for ldmatrix.
// `chunk` counts 16-byte pieces along the head dim (0..31).
template <bool SW>
__device__ __forceinline__ uint32_t tile_offset(int row, int chunk) {
  if (SW) return static_cast<uint32_t>((chunk >> 3) * (PAGE * 128) + row * 128 + (((chunk & 7) ^ (row & 7)) << 4));
  return static_cast<uint32_t>(row * ROW_PITCH + chunk * 16);
}

struct DecodeWarpState {
  uint32_t qb[16][2];  // B fragments of Q^T, one pair per 16-wide slice of head_dim
  float o[16][4];      // O^T accumulators: tile i = dims [16i,16i+16), cols = heads (lane&3)*2,+1
  float m[2];          // running max for heads (lane&3)*2 and +1 (uniform over the lanes that share a head)
  float l[2];          // PER-LANE partial row sums (tokens lane>>2 and lane>>2 + 8 of every page)
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

// Issue the 16 row copies of one K or V tile of a page (`page` points at row 0 of that page and head).
__device__ __forceinline__ void decode_issue_tile(uint8_t* tile, uint64_t* bar, const __nv_bfloat16* page,
                                                  int64_t row_stride, int lane) {
  if (lane == 0) mbar_expect_tx(bar, TILE_TX_BYTES);
  __syncwarp();
  if (lane < PAGE) bulk_g2s(tile + lane * ROW_PITCH, page + lane * row_stride, ROW_BYTES, bar);
}

// Scores and softmax statistics of one staged K tile.  `valid` = leading token rows that belong to the
// sequence (1..16).  Returns the P^T operand fragments (b0, b1) and the rescale factors of the accumulators.
template <bool SW = false>
__device__ __forceinline__ void decode_scores(DecodeWarpState& st, const uint8_t* k_tile, int valid, float scale,
                                              int lane, uint32_t& b0, uint32_t& b1, float& alpha0, float& alpha1) {
  const uint32_t kbase = smem_u32(k_tile);
  // four independent accumulator chains so that consecutive MMAs do not wait on each other
  float sa[4] = {0.f, 0.f, 0.f, 0.f}, sb[4] = {0.f, 0.f, 0.f, 0.f};
  float sc[4] = {0.f, 0.f, 0.f, 0.f}, sd[4] = {0.f, 0.f, 0.f, 0.f};
  {
    const int mi = lane >> 3, r = lane & 7;
    const int arow = r + (mi & 1) * 8, acol = mi >> 1;  // this lane's row and chunk parity inside a 16-dim slice
#pragma unroll
    for (int ks = 0; ks < 16; ks += 4) {
      uint32_t a0[4], a1[4], a2[4], a3[4];
      ldmatrix_x4(a0, kbase + tile_offset<SW>(arow, ks * 2 + acol));
      ldmatrix_x4(a1, kbase + tile_offset<SW>(arow, (ks + 1) * 2 + acol));
      ldmatrix_x4(a2, kbase + tile_offset<SW>(arow, (ks + 2) * 2 + acol));
      ldmatrix_x4(a3, kbase + tile_offset<SW>(arow, (ks + 3) * 2 + acol));
      mma_bf16_16816(sa, a0, st.qb[ks][0], st.qb[ks][1]);
      mma_bf16_16816(sb, a1, st.qb[ks + 1][0], st.qb[ks + 1][1]);
      mma_bf16_16816(sc, a2, st.qb[ks + 2][0], st.qb[ks + 2][1]);
      mma_bf16_16816(sd, a3, st.qb[ks + 3][0], st.qb[ks + 3][1]);
    }
  }
  float s[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) s[i] = (sa[i] + sb[i]) + (sc[i] + sd[i]);
  const int tok = lane >> 2;
  s[0] = (tok < valid) ? s[0] * scale : -INFINITY;
  s[1] = (tok < valid) ? s[1] * scale : -INFINITY;
  s[2] = (tok + 8 < valid) ? s[2] * scale : -INFINITY;
  s[3] = (tok + 8 < valid) ? s[3] * scale : -INFINITY;
  float mx0 = fmaxf(s[0], s[2]), mx1 = fmaxf(s[1], s[3]);
#pragma unroll
  for (int o = 4; o <= 16; o <<= 1) {
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, o));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, o));
  }
  const float m0 = fmaxf(st.m[0], mx0), m1 = fmaxf(st.m[1], mx1);
  alpha0 = __expf(st.m[0] - m0);
  alpha1 = __expf(st.m[1] - m1);
  const float p0 = __expf(s[0] - m0), p1 = __expf(s[1] - m1), p2 = __expf(s[2] - m0), p3 = __expf(s[3] - m1);
  st.l[0] = st.l[0] * alpha0 + (p0 + p2);
  st.l[1] = st.l[1] * alpha1 + (p1 + p3);
  st.m[0] = m0;
  st.m[1] = m1;
  // P^T as the B operand: transpose the two 8x8 bf16 score fragments across the warp
  b0 = movmatrix_trans(pack_bf16(p0, p1));
  b1 = movmatrix_trans(pack_bf16(p2, p3));
}

// O^T = alpha * O^T + V^T . P^T for one staged V tile.
template <bool SW = false>
__device__ __forceinline__ void decode_accumulate(DecodeWarpState& st, uint8_t* v_tile, int valid, uint32_t b0,
                                                  uint32_t b1, float alpha0, float alpha1, int lane) {
  if (valid < PAGE) {
    // rows past the sequence end may hold anything (even NaN bit patterns): clear them so that 0 * garbage
    // cannot poison the accumulators (K garbage is removed by the -inf mask on the scores)
    for (int i = lane; i < (PAGE - valid) * (ROW_BYTES / 16); i += 32) {
      const int r = valid + i / (ROW_BYTES / 16), c = i % (ROW_BYTES / 16);
      *reinterpret_cast<uint4*>(v_tile + tile_offset<SW>(r, c)) = make_uint4(0, 0, 0, 0);
    }
    __syncwarp();
  }
  const uint32_t vbase = smem_u32(v_tile);
  const int mi = lane >> 3, r = lane & 7;
  const int vrow = r + (mi >> 1) * 8, vcol = mi & 1;
  // the running max changes rarely after the first pages: skip the 64 multiplies when no lane needs them
  const bool rescale = __any_sync(0xffffffffu, (alpha0 != 1.f) || (alpha1 != 1.f));
  if (rescale) {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      st.o[i][0] *= alpha0;
      st.o[i][1] *= alpha1;
      st.o[i][2] *= alpha0;
      st.o[i][3] *= alpha1;
    }
  }
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    uint32_t a[4];
    ldmatrix_x4_trans(a, vbase + tile_offset<SW>(vrow, i * 2 + vcol));
    mma_bf16_16816(st.o[i], a, b0, b1);
  }
}

// Row sums are kept per lane; fold them over the 8 token-lanes that share a head (lanes with equal lane&3).
__device__ __forceinline__ void decode_reduce_l(DecodeWarpState& st) {
#pragma unroll
  for (int o = 4; o <= 16; o <<= 1) {
    st.l[0] += __shfl_xor_sync(0xffffffffu, st.l[0], o);
    st.l[1] += __shfl_xor_sync(0xffffffffu, st.l[1], o);
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
