// P = (I + L)^-1 for a strictly lower triangular 64 x 64 fp32 matrix L in shared memory, blocked so that 128 threads
// finish it in a few microseconds: the four 16 x 16 diagonal blocks by forward substitution with the column held in
// registers (one thread per column), then two levels of  P21 = -P22 (L21 P11)  with register tiles.  Used by the
// chunk-64 Gated-DeltaNet kernels (the (I + L) u = beta v solve of triton_kernels/gdn_recurrent_prefill.py:329-342).
// The 16 x 16 and 32 x 32 blocks ABOVE the block diagonal of P are never written: a reader masks i <= t.
#pragma once
#include "common.cuh"

namespace b200 {

constexpr int INV_LP = 68;  // fp32 pitch of the L and P rows: float4 rows, conflict-free for row-per-lane stores
constexpr int INV_TP = 36;  // fp32 pitch of the merge scratch rows
constexpr int INV_SCRATCH_FLOATS = 32 * INV_TP;

// One level of the blocked triangular inverse on the 2N x 2N diagonal block at `base`:  P21 = -P22 (L21 P11).
// merge_a: T = L21 P11, merge_b: P21 = -P22 T; each thread owns one TR x 4 tile (N*N/(4 TR) tiles).  P11 and P22 are
// lower triangular, which bounds the k range; k runs in unrolled groups of eight so that a group's loads are all in
// flight before its FMAs.  Everything is fp32.
template <int N, int TR>
__device__ __forceinline__ void merge_a(const float* Lm, const float* Pm, float* T, int base, int tile) {
  constexpr int TPR = N / 4;
  const int r0 = (tile / TPR) * TR, c0 = (tile % TPR) * 4;
  float acc[TR][4];
#pragma unroll
  for (int i = 0; i < TR; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
  const float* A = Lm + (base + N + r0) * INV_LP + base;
  const float* B = Pm + base * INV_LP + base + c0;
  for (int k0 = c0 & ~7; k0 < N; k0 += 8) {  // P11[k][c] = 0 for k < c
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      const int k = k0 + kk;
      const float4 bq = *reinterpret_cast<const float4*>(B + k * INV_LP);
#pragma unroll
      for (int i = 0; i < TR; ++i) {
        const float av = A[i * INV_LP + k];
        acc[i][0] = fmaf(av, bq.x, acc[i][0]);
        acc[i][1] = fmaf(av, bq.y, acc[i][1]);
        acc[i][2] = fmaf(av, bq.z, acc[i][2]);
        acc[i][3] = fmaf(av, bq.w, acc[i][3]);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < TR; ++i)
    *reinterpret_cast<float4*>(T + (r0 + i) * INV_TP + c0) = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
}
template <int N, int TR>
__device__ __forceinline__ void merge_b(float* Pm, const float* T, int base, int tile) {
  constexpr int TPR = N / 4;
  const int r0 = (tile / TPR) * TR, c0 = (tile % TPR) * 4;
  float acc[TR][4];
#pragma unroll
  for (int i = 0; i < TR; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
  const float* A = Pm + (base + N + r0) * INV_LP + base + N;
  for (int k0 = 0; k0 <= r0 + TR - 1; k0 += 8) {  // P22[r][k] = 0 for k > r
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      const int k = k0 + kk;
      const float4 bq = *reinterpret_cast<const float4*>(T + k * INV_TP + c0);
#pragma unroll
      for (int i = 0; i < TR; ++i) {
        const float av = A[i * INV_LP + k];
        acc[i][0] = fmaf(-av, bq.x, acc[i][0]);
        acc[i][1] = fmaf(-av, bq.y, acc[i][1]);
        acc[i][2] = fmaf(-av, bq.z, acc[i][2]);
        acc[i][3] = fmaf(-av, bq.w, acc[i][3]);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < TR; ++i)
    *reinterpret_cast<float4*>(Pm + (base + N + r0 + i) * INV_LP + base + c0) =
        make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
}

// Called by threads 0..127 of the CTA (tid = their index), all of them; Lm and Pm are [64][INV_LP], Tm is
// INV_SCRATCH_FLOATS of scratch.  The five internal barriers are named barrier 3 over those 128 threads; the caller
// synchronises before (L complete) and after (P complete) by its own means.
__device__ __forceinline__ void blocked_inverse64(const float* Lm, float* Pm, float* Tm, int tid) {
  if (tid < 64) {
    const int blk = tid >> 4, j = tid & 15;
    const float* lb = Lm + (16 * blk) * INV_LP + 16 * blk;
    float xx[16];
#pragma unroll
    for (int r = 0; r < 16; ++r) {
      float a0 = (r == j) ? 1.f : 0.f, a1 = 0.f;
#pragma unroll
      for (int i = 0; i < r; ++i) {
        if (i & 1) a1 = fmaf(-lb[r * INV_LP + i], xx[i], a1);
        else a0 = fmaf(-lb[r * INV_LP + i], xx[i], a0);
      }
      xx[r] = a0 + a1;
    }
#pragma unroll
    for (int r = 0; r < 16; ++r) Pm[(16 * blk + r) * INV_LP + 16 * blk + j] = xx[r];  // after the loop: no aliasing stalls
  }
  named_barrier(3, 128);
  if (tid < 64) merge_a<16, 2>(Lm, Pm, Tm + (tid >> 5) * 16 * INV_TP, 32 * (tid >> 5), tid & 31);
  named_barrier(3, 128);
  if (tid < 64) merge_b<16, 2>(Pm, Tm + (tid >> 5) * 16 * INV_TP, 32 * (tid >> 5), tid & 31);
  named_barrier(3, 128);
  merge_a<32, 2>(Lm, Pm, Tm, 0, tid);
  named_barrier(3, 128);
  merge_b<32, 2>(Pm, Tm, 0, tid);
}

}  // namespace b200
