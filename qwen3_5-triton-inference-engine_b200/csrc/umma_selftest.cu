// Self-test of the sm_100a building blocks in umma.cuh: one CTA loads two bf16 operand tiles with tensor-map TMA
// (128-byte swizzle), multiplies them with tcgen05.mma into tensor memory and writes the fp32 result back.
//   mode 0: C[128 x 64]  = A[128 x 256] . B[64 x 256]^T     (B is K-major: the QK^T shape of prefill attention)
//   mode 1: C[128 x 256] = A[128 x 64]  . B[64 x 256]       (B is MN-major: the P.V shape)
//   mode 2: the same product with A written to TENSOR MEMORY by the threads (two bf16 per 32-bit column) and used as
//           the MMA's A operand from there (the form in which prefill attention hands P to the PV product)
// It exists so that descriptor or layout mistakes show up in a 10-microsecond kernel with a known answer instead
// of inside the attention kernels; tests/test_gpu_umma.py compares it with torch.matmul.
#include "b200_attn.h"
#include "umma.cuh"

namespace b200 {

bool encode_map_bf16_sw128(CUtensorMap* map, const void* base, int rank, const uint64_t* dims,
                           const uint64_t* strides_bytes, const uint32_t* box) {
  typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                               const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static EncodeFn encode = nullptr;
  if (!encode) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess || fn == nullptr) {
      cudaGetLastError();
      return false;
    }
    encode = reinterpret_cast<EncodeFn>(fn);
  }
  if (rank < 3 || rank > 5 || dims[0] != 64 || box[0] != 64 || (reinterpret_cast<uintptr_t>(base) & 15) != 0) return false;
  cuuint64_t d[5], st[4];
  cuuint32_t bx[5], es[5];
  for (int i = 0; i < rank; ++i) {
    d[i] = dims[i];
    bx[i] = box[i];
    es[i] = 1;
    if (i + 1 < rank) {
      if (strides_bytes[i] % 16 != 0) return false;
      st[i] = strides_bytes[i];
    }
  }
  return encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, static_cast<cuuint32_t>(rank), const_cast<void*>(base), d, st, bx,
                es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool encode_tile_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t row_stride_bytes,
                     uint32_t box_rows, uint32_t box_blocks) {
  if (cols % 64 != 0) return false;
  const uint64_t dims[3] = {64, rows, cols / 64};
  const uint64_t strides[2] = {row_stride_bytes, 128};
  const uint32_t box[3] = {64, box_rows, box_blocks};
  return encode_map_bf16_sw128(map, base, 3, dims, strides, box);
}

constexpr int ST_A_BYTES = 128 * 256 * 2;  // largest A tile (mode 0)
constexpr int ST_B_BYTES = 64 * 256 * 2;
constexpr int ST_SMEM = ST_A_BYTES + ST_B_BYTES + 1024;

__global__ void __launch_bounds__(128, 1)
umma_selftest_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                     float* __restrict__ c, int mode, int* __restrict__ err) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ uint64_t bar_tma, bar_mma;
  __shared__ uint32_t tmem_slot;
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* a_s = smem;
  uint8_t* b_s = smem + ST_A_BYTES;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n = mode == 0 ? 64 : 256;
  constexpr uint32_t TMEM_COLS = 512;  // C in [0,256); mode 2 keeps A in [256,288)

  if (warp == 0) tmem_alloc(&tmem_slot, TMEM_COLS);
  if (tid == 0) {
    mbar_init(&bar_tma, 1);
    mbar_init(&bar_mma, 1);
    mbar_fence_init();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = tmem_slot;

  if (tid == 0) {
    if (mode == 0) {
      mbar_expect_tx(&bar_tma, 128 * 256 * 2 + 64 * 256 * 2);
      tma_load_3d(a_s, &map_a, 0, 0, 0, &bar_tma);  // {64 cols, 128 rows, 4 blocks}
      tma_load_3d(b_s, &map_b, 0, 0, 0, &bar_tma);  // {64 cols, 64 rows, 4 blocks}
    } else {
      mbar_expect_tx(&bar_tma, 128 * 64 * 2 + 64 * 256 * 2);
      tma_load_3d(a_s, &map_a, 0, 0, 0, &bar_tma);  // {64 cols, 128 rows, 1 block}
      tma_load_3d(b_s, &map_b, 0, 0, 0, &bar_tma);  // {64 cols, 64 rows, 4 blocks}
    }
  }
  bool ok = mbar_wait_bounded(&bar_tma, 0);
  if (mode == 2) {
    // row `tid` of A: 64 bf16 = 32 packed words, read from the swizzled tile and stored to TMEM columns [256, 288)
    uint32_t w[32];
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const uint4 v = *reinterpret_cast<const uint4*>(a_s + tid * 128 + ((c ^ (tid & 7)) << 4));
      w[c * 4] = v.x; w[c * 4 + 1] = v.y; w[c * 4 + 2] = v.z; w[c * 4 + 3] = v.w;
    }
    tmem_st32(tmem + (static_cast<uint32_t>(warp * 32) << 16) + 256, w);
    tmem_st_wait();
    tc_fence_before_sync();
    __syncthreads();
  }
  if (ok && tid == 0) {
    tc_fence_after_sync();
    if (mode == 0) {
      // K-major A [128 x 256] and K-major B [64 x 256]: 16 steps of K=16 (32 bytes inside a 128-byte block row)
      const uint32_t idesc = idesc_bf16_f32(128, 64, false, false);
      for (int ks = 0; ks < 16; ++ks) {
        const uint32_t a_addr = smem_u32(a_s) + (ks >> 2) * (128 * 128) + (ks & 3) * 32;
        const uint32_t b_addr = smem_u32(b_s) + (ks >> 2) * (64 * 128) + (ks & 3) * 32;
        umma_ss(tmem, smem_desc_sw128(a_addr, 16, 1024), smem_desc_sw128(b_addr, 16, 1024), idesc, ks > 0);
      }
    } else if (mode == 2) {
      const uint32_t idesc = idesc_bf16_f32(128, 256, false, true);
      for (int kt = 0; kt < 4; ++kt)
        umma_ts_leader(tmem, tmem + 256 + kt * 8, smem_desc_sw128(smem_u32(b_s) + kt * 2048, 64 * 128, 1024), idesc,
                       kt > 0, true);
    } else {
      // K-major A [128 x 64] and MN-major B [64 (K) x 256 (N)]: 4 steps of K=16 rows of B (2048 bytes apart)
      const uint32_t idesc = idesc_bf16_f32(128, 256, false, true);
      for (int kt = 0; kt < 4; ++kt) {
        const uint32_t a_addr = smem_u32(a_s) + kt * 32;
        const uint32_t b_addr = smem_u32(b_s) + kt * 2048;
        umma_ss(tmem, smem_desc_sw128(a_addr, 16, 1024), smem_desc_sw128(b_addr, 64 * 128, 1024), idesc, kt > 0);
      }
    }
    umma_commit(&bar_mma);
  }
  if (ok) ok = mbar_wait_bounded(&bar_mma, 0);
  if (ok) {
    tc_fence_after_sync();
    const int row = warp * 32 + lane;
    for (int c0 = 0; c0 < n; c0 += 32) {
      uint32_t r[32];
      tmem_ld32(tmem + (static_cast<uint32_t>(warp * 32) << 16) + c0, r);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; ++j) c[row * n + c0 + j] = __uint_as_float(r[j]);
    }
  } else if (tid == 0) {
    atomicExch(err, 1);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, TMEM_COLS);
}

// The give-up path of every staged copy in this library, exercised on purpose: an mbarrier is armed for bytes that no
// copy will ever deliver, one warp waits for it with a small poll limit, the wait returns false, the kernel records that
// in the error word, leaves `sentinel` untouched (what a real kernel does with its outputs on this path) and returns.
// Nothing is in flight when it ends; the context stays usable.
__global__ void wait_timeout_selftest_kernel(int* err, int* sentinel, uint32_t polls) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    mbar_fence_init();
    mbar_expect_tx(&bar, 16);  // the one arrival is made, the 16 bytes never come
  }
  __syncwarp();
  const bool ok = mbar_wait_bounded(&bar, 0, polls);
  if (threadIdx.x == 0) {
    if (ok) *sentinel = 1;  // would mean the wait did NOT run out
    else atomicExch(err, 1);
  }
}

}  // namespace b200

using namespace b200;

extern "C" int b200_selftest_wait_timeout(int32_t* sentinel, b200_stream_t stream) {
  int* err = wait_timeout_flag();
  if (!err) return fail(ERR_RUNTIME, "selftest_wait_timeout: no error flag");
  B200_REQUIRE(sentinel != nullptr, "selftest_wait_timeout: sentinel is NULL");
  wait_timeout_selftest_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(err, sentinel, 1u << 10);
  return check_launch("selftest_wait_timeout");
}

extern "C" int b200_selftest_umma(int32_t mode, const void* a, const void* b, float* c, b200_stream_t stream) {
  B200_REQUIRE(mode >= 0 && mode <= 2, "selftest_umma: mode must be 0, 1 or 2");
  CUtensorMap map_a, map_b;
  bool ok;
  if (mode == 0) {
    ok = encode_tile_map(&map_a, a, 128, 256, 512, 128, 4) && encode_tile_map(&map_b, b, 64, 256, 512, 64, 4);
  } else {
    ok = encode_tile_map(&map_a, a, 128, 64, 128, 128, 1) && encode_tile_map(&map_b, b, 64, 256, 512, 64, 4);
  }
  if (!ok) return fail(ERR_RUNTIME, "selftest_umma: cuTensorMapEncodeTiled is unavailable or refused the tile map");
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    if (cudaFuncSetAttribute(umma_selftest_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, ST_SMEM) != cudaSuccess)
      return fail(ERR_RUNTIME, "selftest_umma: cannot raise dynamic shared memory to %d", ST_SMEM);
    configured[dev] = true;
  }
  int* err = wait_timeout_flag();
  if (!err) return fail(ERR_RUNTIME, "selftest_umma: no error flag");
  umma_selftest_kernel<<<1, 128, ST_SMEM, reinterpret_cast<cudaStream_t>(stream)>>>(map_a, map_b, c, mode, err);
  return check_launch("selftest_umma");
}
