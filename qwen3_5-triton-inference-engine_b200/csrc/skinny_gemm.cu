// Weight-streaming GEMM for decode batches:  Y[M, N] = X[M, K] . W[N, K]^T  with M <= 32 rows (one token per
// sequence), bf16 in / bf16 out, fp32 accumulation.  Replaces triton_kernels/gemm_2d.py for the decode-step projections
// whose input width is the model's hidden size; the reference's own note is that these GEMVs are about half of a
// decode step (README-EN.md:116).
//
// The product is HBM-bound on W (M is tiny), so the kernel is built like the decode-attention kernels: X is staged once
// per CTA in shared memory (one bulk copy per row), every warp streams rows of W through a private ring of 4 KiB tiles
// (tensor-map TMA, 128-byte swizzle -> conflict-free ldmatrix, one mbarrier per tile, no cluster multicast), and
// multiplies with mma.sync m16n8k16 taking the W rows as the MMA M dimension and the batch as N (M <= 32 is far too
// thin for a tcgen05 tile).  CTAs walk the row blocks persistently, so X is read once per CTA however large N is.
// Every wait is bounded.
//
// Two forms.  Plain: a warp's tile is 16 consecutive rows of W (one box {64 k, 16 rows, 2 k-blocks}), a CTA covers 64
// outputs with four row groups of two warps each (the even and the odd k tiles).  SwiGLU (W = [gate rows | up rows], the fused gate/up projection followed by
// triton_kernels/swiglu.py): a warp's tile is 8 gate rows stacked on the 8 matching up rows (two boxes of 8 rows), so the
// accumulator fragment of a thread holds gate_j (row r) and up_j (row r + 8) of the same output j and the activation is
// applied in registers; a CTA covers 32 outputs.
#include "b200_attn.h"
#include "umma.cuh"

#include <mutex>

namespace b200 {

constexpr int SG_WARPS = 4;
constexpr int SG_THREADS = SG_WARPS * 32;
constexpr int SG_ROWS = 16 * SG_WARPS;   // outputs per CTA step, plain form (8 * SG_WARPS in the SwiGLU form)
constexpr int SG_TILE_K = 128;           // k elements per tile: two swizzled blocks of [16 rows][64 k] bf16
constexpr int SG_TILE_BYTES = 2 * 16 * 128;
constexpr int SG_RING = 8;                        // tiles in flight per warp
constexpr int SG_RING_BYTES = SG_RING * SG_TILE_BYTES;
constexpr int SG_KSPLIT = 2;                      // K = 1280 or less: warps per row group, alternating k tiles
constexpr int SG_STD_WARPS = SG_WARPS * SG_KSPLIT;
constexpr int SG_STD_THREADS = SG_STD_WARPS * 32;
constexpr int SG_STD_RING = SG_RING / SG_KSPLIT;  // the same bytes in flight per CTA
constexpr int SG_PART_BYTES = 16 * SG_WARPS * 32 * 4;
constexpr int SG_MAX_M = 32;
constexpr int SG_MAX_K = 1280;           // X staging: 32 x (K*2 + 16) bytes next to 128 KiB of weight rings

struct SkinnyGemmParams {
  const __nv_bfloat16* x;  // [M, K]
  __nv_bfloat16* y;        // [M, N]
  int64_t x_stride, y_stride;
  int* err;
  int m, n, k, row_blocks, overlap, up_row0;  // n: outputs; up_row0: first W row of the `up` half (SwiGLU form)
  // arg-max form: ids[b] = argmax_n y[b, n] instead of y (keys / counter: zero-filled workspace, left zero)
  int64_t* ids;
  unsigned long long* keys;
  int* counter;
};

template <bool SWIGLU, bool ARGMAX>
__global__ void __launch_bounds__(SG_STD_THREADS, 1)
skinny_gemm_kernel(const __grid_constant__ SkinnyGemmParams p, const __grid_constant__ CUtensorMap map_w) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  constexpr int SLOT_BYTES = SG_TILE_BYTES;
  constexpr int RING = SG_STD_RING;
  constexpr int OUT = SWIGLU ? 8 * SG_WARPS : SG_ROWS;  // outputs per CTA step
  __shared__ uint64_t bars[SG_STD_WARPS][RING];
  __shared__ uint64_t bar_x;
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // warps wr and wr + 4 share the rows of group wr and take the even / the odd k tiles: a warp's k steps are a chain of
  // dependent ldmatrix + MMA, so two short chains per row group finish in half the time of one long one
  const int wr = warp & (SG_WARPS - 1), kh = warp / SG_WARPS;
  uint8_t* ring = smem + warp * (RING * SLOT_BYTES);
  uint8_t* stage = smem + SG_WARPS * SG_RING_BYTES;                    // [32 batch][OUT] bf16 output staging, <= 4 KiB
  float* part = reinterpret_cast<float*>(stage + SG_MAX_M * SG_ROWS * 2);  // [16][4 groups x 32 lanes]: odd-tile sums
  uint8_t* xs = reinterpret_cast<uint8_t*>(part) + SG_PART_BYTES;      // [32][x_pitch] bf16
  const int x_pitch = p.k * 2 + 16;                                    // bytes; the 16 shift the banks row by row
  const int k_tiles = p.k / SG_TILE_K;

  if (lane == 0) {
    for (int s = 0; s < RING; ++s) mbar_init(&bars[warp][s], 1);
    if (warp == 0) mbar_init(&bar_x, 1);
    mbar_fence_init();
  }
  // my tiles: row block rb = blockIdx.x, + gridDim.x, ...; tile index t counts (row block, k tile) pairs
  const int my_blocks = (p.row_blocks - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x);
  const int my_kt = (k_tiles - kh + SG_KSPLIT - 1) / SG_KSPLIT;  // k tiles kh, kh + 2, ... of every row block
  const int total_tiles = my_blocks * my_kt;
  __syncwarp();
  auto issue = [&](int t) {
    const int rb = blockIdx.x + (t / my_kt) * gridDim.x, kt = kh + SG_KSPLIT * (t % my_kt);
    const int slot = t % RING;
    mbar_expect_tx(&bars[warp][slot], SLOT_BYTES);
    if (SWIGLU) {  // map_w has 8-row boxes: gate rows to the first half of the tile, up rows to the second
      tma_load_3d(ring + slot * SLOT_BYTES, &map_w, 0, rb * OUT + wr * 8, kt * 2, &bars[warp][slot]);
      tma_load_3d(ring + slot * SLOT_BYTES + SG_TILE_BYTES / 2, &map_w, 0, p.up_row0 + rb * OUT + wr * 8, kt * 2,
                  &bars[warp][slot]);
    } else {
      tma_load_3d(ring + slot * SLOT_BYTES, &map_w, 0, rb * OUT + wr * 16, kt * 2, &bars[warp][slot]);
    }
  };
  auto stage_x = [&]() {  // warp 0: one bulk copy per row of X
    if (lane == 0) mbar_expect_tx(&bar_x, static_cast<uint32_t>(p.m) * p.k * 2);
    __syncwarp();
    if (lane < p.m) bulk_g2s(xs + lane * x_pitch, p.x + static_cast<int64_t>(lane) * p.x_stride, p.k * 2, &bar_x);
  };
  // Started early, the weights are requested while the predecessor runs and X after it.  In plain stream order X goes
  // first: requested behind 128 KiB of weight tiles it would arrive behind them.
  const bool early = (p.overlap & OVERLAP_START) != 0;
  if (p.overlap & OVERLAP_TRIGGER) pdl_trigger();
  if (!early && warp == 0) stage_x();
  if (lane == 0) {
    for (int t = 0; t < RING && t < total_tiles; ++t) issue(t);  // weights: independent of the predecessor
  }
  pdl_wait();  // X is the predecessor's output
  if (early && warp == 0) stage_x();
  for (int i = tid; i < (SG_MAX_M - p.m) * (p.k >> 3); i += SG_STD_THREADS) {  // rows beyond M are zero
    const int r = p.m + i / (p.k >> 3), c = i % (p.k >> 3);
    *reinterpret_cast<uint4*>(xs + r * x_pitch + c * 16) = make_uint4(0, 0, 0, 0);
  }
  __syncthreads();  // bar_x is initialised for everybody, the zero rows are in place
  bool ok = mbar_wait_bounded(&bar_x, 0);

  const uint32_t xs_base = smem_u32(xs);
  // ldmatrix lane addresses: A (W tile) row = lane % 16, chunk parity = lane / 16;
  //                          B (X) row = (lane & 7) + 8 * (lane >> 4) inside a 16-row pair, k half = (lane >> 3) & 1
  const int a_row = lane & 15, a_par = lane >> 4;
  const uint32_t b_lane = static_cast<uint32_t>(((lane & 7) + ((lane >> 4) << 3)) * x_pitch + ((lane >> 3) & 1) * 16);
  // arg-max form: this thread's running best over its rows, per batch column (8 columns: nt * 2 + (j & 1))
  float best_v[8];
  uint32_t best_i[8];
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    best_v[c] = -INFINITY;
    best_i[c] = 0xffffffffu;
  }
  int t = 0;
  for (int blk = 0; blk < my_blocks; ++blk) {  // a failed wait clears `ok`; the loop then only keeps its barriers
    const int rb = blockIdx.x + blk * gridDim.x;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
    for (int kt = kh; kt < k_tiles && ok; kt += SG_KSPLIT, ++t) {
      const int slot = t % RING;
      if (!mbar_wait_bounded(&bars[warp][slot], (t / RING) & 1)) {
        ok = false;
        break;
      }
      const uint32_t tile = smem_u32(ring + slot * SLOT_BYTES);
#pragma unroll
      for (int ks = 0; ks < SG_TILE_K / 16; ++ks) {
        uint32_t a[4], b01[4], b23[4];
        // plain: [k-block][16 rows][128 B]; SwiGLU: [gate | up][k-block][8 rows][128 B]; 16-byte chunks XOR-swizzled by row
        const uint32_t a_off = (SWIGLU ? (a_row >> 3) * (SG_TILE_BYTES / 2) + (ks >> 2) * (8 * 128) + (a_row & 7) * 128
                                       : (ks >> 2) * (16 * 128) + a_row * 128) +
                               ((((ks & 3) * 2 + a_par) ^ (a_row & 7)) << 4);
        const uint32_t xk = xs_base + b_lane + (kt * SG_TILE_K + ks * 16) * 2;
        ldmatrix_x4(b01, xk);                   // batch rows 0-15: (b0, b1) of n8 tiles 0 and 1
        ldmatrix_x4(b23, xk + 16 * x_pitch);    // batch rows 16-31
        ldmatrix_x4(a, tile + a_off);
        mma_bf16_16816(acc[0], a, b01[0], b01[1]);
        mma_bf16_16816(acc[1], a, b01[2], b01[3]);
        mma_bf16_16816(acc[2], a, b23[0], b23[1]);
        mma_bf16_16816(acc[3], a, b23[2], b23[3]);
      }
      __syncwarp();  // every lane has read the tile: its slot can take the tile RING ahead
      if (lane == 0 && t + RING < total_tiles) issue(t + RING);
    }
    // the odd-tile warps hand their sums to the even-tile warps of the same row group
    if (kh == 1) {
#pragma unroll
      for (int i = 0; i < 16; ++i) part[i * (SG_WARPS * 32) + wr * 32 + lane] = acc[i >> 2][i & 3];
    }
    __syncthreads();  // (also: the previous block's staging has been written out)
    // acc[nt]: rows (tile row = lane/4, +8), cols (batch = nt*8 + (lane%4)*2, +1)  ->  stage[batch][output] -> Y
    if (kh == 0) {
#pragma unroll
      for (int i = 0; i < 16; ++i) acc[i >> 2][i & 3] += part[i * (SG_WARPS * 32) + wr * 32 + lane];
    }
    if (ARGMAX) {
      if (kh == 0) {
        // rows ascend with the row block and, inside it, from fragment row r to r + 8: strict > keeps the lowest index
        const uint32_t n_lo = static_cast<uint32_t>(rb * OUT + wr * 16 + (lane >> 2));
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int c = nt * 2 + (j & 1);
            const uint32_t n = n_lo + (j >= 2 ? 8u : 0u);
            if (n < static_cast<uint32_t>(p.n) && (acc[nt][j] > best_v[c] || best_i[c] == 0xffffffffu)) {
              best_v[c] = acc[nt][j];
              best_i[c] = n;
            }
          }
      }
      __syncthreads();  // `part` may be rewritten by the next row block
      continue;
    }
    if (kh == 0) {
      __nv_bfloat16* st = reinterpret_cast<__nv_bfloat16*>(stage);
      const int bc = (lane & 3) * 2;
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        if (SWIGLU) {
          // rows r and r + 8 of the tile are gate_j and up_j; the projection is a bf16 tensor in the reference
          const int j = wr * 8 + (lane >> 2);
          const float g0 = round_bf16(acc[nt][0]), g1 = round_bf16(acc[nt][1]);
          const float u0 = round_bf16(acc[nt][2]), u1 = round_bf16(acc[nt][3]);
          st[(nt * 8 + bc) * OUT + j] = __float2bfloat16_rn(g0 / (1.0f + expf(-g0)) * u0);
          st[(nt * 8 + bc + 1) * OUT + j] = __float2bfloat16_rn(g1 / (1.0f + expf(-g1)) * u1);
        } else {
          const int nr = wr * 16 + (lane >> 2);
          st[(nt * 8 + bc) * OUT + nr] = __float2bfloat16_rn(acc[nt][0]);
          st[(nt * 8 + bc + 1) * OUT + nr] = __float2bfloat16_rn(acc[nt][1]);
          st[(nt * 8 + bc) * OUT + nr + 8] = __float2bfloat16_rn(acc[nt][2]);
          st[(nt * 8 + bc + 1) * OUT + nr + 8] = __float2bfloat16_rn(acc[nt][3]);
        }
      }
    }
    __syncthreads();
    for (int i = tid; i < SG_MAX_M * (OUT / 8); i += SG_STD_THREADS) {
      const int r = i / (OUT / 8), c = i % (OUT / 8);
      const int n0 = rb * OUT + c * 8;
      if (r < p.m && n0 < p.n)  // N is a multiple of 8: a 16-byte chunk is inside or outside as a whole
        *reinterpret_cast<uint4*>(p.y + static_cast<int64_t>(r) * p.y_stride + n0) =
            *reinterpret_cast<const uint4*>(stage + (r * OUT + c * 8) * 2);
    }
  }
  if (ARGMAX) {
    // lanes that share lane % 4 hold the same batch columns: fold them, then the four row groups, then the CTAs
    unsigned long long* keybuf = reinterpret_cast<unsigned long long*>(part);  // [4 row groups][32 batch]
    if (kh == 0) {
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        unsigned long long key = best_i[c] == 0xffffffffu ? 0ull : argmax_key(best_v[c], best_i[c]);
#pragma unroll
        for (int o = 4; o <= 16; o <<= 1) {
          const unsigned long long other = __shfl_xor_sync(0xffffffffu, key, o);
          key = other > key ? other : key;
        }
        if (lane < 4) keybuf[wr * SG_MAX_M + (c >> 1) * 8 + lane * 2 + (c & 1)] = key;
      }
    }
    __syncthreads();
    if (warp == 0) {
      if (lane < p.m && ok) {
        unsigned long long key = keybuf[lane];
#pragma unroll
        for (int w = 1; w < SG_WARPS; ++w) key = keybuf[w * SG_MAX_M + lane] > key ? keybuf[w * SG_MAX_M + lane] : key;
        atomicMax(p.keys + lane, key);
      }
      __threadfence();
      __syncwarp();
      int last = 0;
      if (lane == 0) last = (atomicAdd(p.counter, 1) == static_cast<int>(gridDim.x) - 1);
      last = __shfl_sync(0xffffffffu, last, 0);
      if (last) {  // every CTA's keys are in: unpack the ids and leave the workspace zero for the next launch
        __threadfence();
        if (lane < p.m) {
          const unsigned long long top = atomicExch(p.keys + lane, 0ull);
          p.ids[lane] = static_cast<int64_t>(0xffffffffu - static_cast<uint32_t>(top & 0xffffffffull));
        }
        if (lane == 0) *p.counter = 0;
      }
    }
  }
  if (!ok) {
    if (lane == 0) atomicExch(p.err, 1);
    // let this warp's copies in flight land before the shared memory goes away
    for (int s = 0; s < RING; ++s) mbar_wait_bounded(&bars[warp][s], 0, 1u << 12);
  }
}

// ------------------------------------------------------------------------------------------------ wide-K form
// Projections back to the hidden size (out / o / down projection: N = hidden, K = 2048 .. 3584 and more) have few
// output rows and long ones.  A CTA owns 16 outputs (one MMA M tile) and its four warps split K: warp w streams the
// 4 KiB tiles kt = w, w + 4, ... of those 16 rows, accumulates its own [16 x 32] product and the four partial sums meet
// in shared memory (fixed order, so the result is deterministic).  X no longer fits next to the rings, so it is staged
// in chunks of at most 1024 k, double-buffered: the last warp to leave a chunk (a counter in shared memory, nobody
// waits) requests the chunk after the next into the buffer that just became free.
constexpr int WK_RING = 5;                // W tiles in flight per warp
constexpr int WK_CHUNK_MAX = 1024;        // k elements of X per staged chunk
constexpr int WK_ROWS = 16;               // outputs per CTA step
constexpr int WK_MAX_K = 16384;
constexpr int WK_X_PITCH_MAX = WK_CHUNK_MAX * 2 + 16;
constexpr int WK_SMEM = SG_WARPS * WK_RING * SG_TILE_BYTES + SG_WARPS * WK_ROWS * SG_MAX_M * 4 +
                        2 * SG_MAX_M * WK_X_PITCH_MAX + 1024;
static_assert(WK_SMEM <= 227 * 1024, "weight rings + two X chunks must fit the 227 KiB a CTA may use");

struct WideKParams {
  const __nv_bfloat16* x;  // [M, K]
  __nv_bfloat16* y;        // [M, N]
  int64_t x_stride, y_stride;
  int* err;
  int m, n, k, row_blocks, overlap, chunk_k, n_chunks;
};

__global__ void __launch_bounds__(SG_THREADS, 1)
skinny_gemm_widek_kernel(const __grid_constant__ WideKParams p, const __grid_constant__ CUtensorMap map_w) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ uint64_t bars[SG_WARPS][WK_RING];
  __shared__ uint64_t bar_x[2];
  __shared__ int x_left[2];  // warps that have left the chunk in buffer 0 / 1 (counts up, never reset)
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  uint8_t* ring = smem + warp * WK_RING * SG_TILE_BYTES;
  float* red = reinterpret_cast<float*>(smem + SG_WARPS * WK_RING * SG_TILE_BYTES);   // [4 warps][32 batch][16 rows]
  uint8_t* xs = reinterpret_cast<uint8_t*>(red) + SG_WARPS * WK_ROWS * SG_MAX_M * 4;  // [2][32][x_pitch]
  const int x_pitch = p.chunk_k * 2 + 16;
  const int x_buf_bytes = SG_MAX_M * x_pitch;
  const int k_tiles = p.k / SG_TILE_K, chunk_tiles = p.chunk_k / SG_TILE_K;

  if (tid == 0) {
    for (int w = 0; w < SG_WARPS; ++w)
      for (int s = 0; s < WK_RING; ++s) mbar_init(&bars[w][s], 1);
    mbar_init(&bar_x[0], 1);
    mbar_init(&bar_x[1], 1);
    x_left[0] = x_left[1] = 0;
    mbar_fence_init();
  }
  const int my_blocks = (p.row_blocks - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x);
  const int my_tiles = k_tiles > warp ? (k_tiles - warp + SG_WARPS - 1) / SG_WARPS : 0;  // per row block, this warp
  const int total_tiles = my_blocks * my_tiles;
  const int total_chunks = my_blocks * p.n_chunks;
  __syncthreads();
  auto issue = [&](int t) {  // lane 0: tile t of this warp = (row block t / my_tiles, k tile warp + 4 * (t % my_tiles))
    const int rb = blockIdx.x + (t / my_tiles) * gridDim.x, kt = warp + SG_WARPS * (t % my_tiles);
    const int slot = t % WK_RING;
    mbar_expect_tx(&bars[warp][slot], SG_TILE_BYTES);
    tma_load_3d(ring + slot * SG_TILE_BYTES, &map_w, 0, rb * WK_ROWS, kt * 2, &bars[warp][slot]);
  };
  // chunk q of this CTA's chunk stream (row block q / n_chunks, k range (q % n_chunks) * chunk_k ...) -> buffer q & 1
  auto stage_x = [&](int q) {  // a whole warp
    const int buf = q & 1, c = q % p.n_chunks;
    if (lane == 0) mbar_expect_tx(&bar_x[buf], static_cast<uint32_t>(p.m) * p.chunk_k * 2);
    __syncwarp();
    if (lane < p.m)
      bulk_g2s(xs + buf * x_buf_bytes + lane * x_pitch, p.x + static_cast<int64_t>(lane) * p.x_stride + c * p.chunk_k,
               p.chunk_k * 2, &bar_x[buf]);
  };
  if (p.overlap & OVERLAP_TRIGGER) pdl_trigger();
  if (lane == 0) {
    for (int t = 0; t < WK_RING && t < total_tiles; ++t) issue(t);  // weights: independent of the predecessor
  }
  pdl_wait();  // X is the predecessor's output
  for (int i = tid; i < 2 * (SG_MAX_M - p.m) * (p.chunk_k >> 3); i += SG_THREADS) {  // rows beyond M are zero
    const int per_buf = (SG_MAX_M - p.m) * (p.chunk_k >> 3);
    const int buf = i / per_buf, j = i % per_buf;
    const int r = p.m + j / (p.chunk_k >> 3), c = j % (p.chunk_k >> 3);
    *reinterpret_cast<uint4*>(xs + buf * x_buf_bytes + r * x_pitch + c * 16) = make_uint4(0, 0, 0, 0);
  }
  if (warp == 0) {
    stage_x(0);
    if (total_chunks > 1) stage_x(1);
  }
  __syncthreads();  // the zero rows are in place

  const int a_row = lane & 15, a_par = lane >> 4;
  const uint32_t b_lane = static_cast<uint32_t>(((lane & 7) + ((lane >> 4) << 3)) * x_pitch + ((lane >> 3) & 1) * 16);
  bool ok = true;
  int t = 0;
  // leave chunk q: the last of the four warps to do so requests chunk q + 2 into the buffer that is now free
  auto leave_chunk = [&](int q) {
    int last = 0;
    if (lane == 0) last = ((atomicAdd(&x_left[q & 1], 1) & (SG_WARPS - 1)) == SG_WARPS - 1);
    last = __shfl_sync(0xffffffffu, last, 0);
    if (last && q + 2 < total_chunks) stage_x(q + 2);
  };
  for (int blk = 0; blk < my_blocks; ++blk) {
    const int rb = blockIdx.x + blk * gridDim.x;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
    int cur = -1;  // chunk (within the row block) whose X this warp is reading
    for (int kt = warp; kt < k_tiles; kt += SG_WARPS, ++t) {
      const int c = kt / chunk_tiles;
      while (cur < c) {  // move on to the chunk of this tile, leaving the ones in between
        if (cur >= 0) leave_chunk(blk * p.n_chunks + cur);
        ++cur;
      }
      const int q = blk * p.n_chunks + c;
      if (ok && !mbar_wait_bounded(&bar_x[q & 1], (q >> 1) & 1)) ok = false;
      const int slot = t % WK_RING;
      if (ok && !mbar_wait_bounded(&bars[warp][slot], (t / WK_RING) & 1)) ok = false;
      if (ok) {
        const uint32_t tile = smem_u32(ring + slot * SG_TILE_BYTES);
        const uint32_t xk0 = smem_u32(xs + (q & 1) * x_buf_bytes) + b_lane + ((kt - c * chunk_tiles) * SG_TILE_K) * 2;
#pragma unroll
        for (int ks = 0; ks < SG_TILE_K / 16; ++ks) {
          uint32_t a[4], b01[4], b23[4];
          const uint32_t a_off = (ks >> 2) * (16 * 128) + a_row * 128 + ((((ks & 3) * 2 + a_par) ^ (a_row & 7)) << 4);
          ldmatrix_x4(b01, xk0 + ks * 32);
          ldmatrix_x4(b23, xk0 + ks * 32 + 16 * x_pitch);
          ldmatrix_x4(a, tile + a_off);
          mma_bf16_16816(acc[0], a, b01[0], b01[1]);
          mma_bf16_16816(acc[1], a, b01[2], b01[3]);
          mma_bf16_16816(acc[2], a, b23[0], b23[1]);
          mma_bf16_16816(acc[3], a, b23[2], b23[3]);
        }
      }
      __syncwarp();  // every lane has read the tile: its slot can take the tile WK_RING ahead
      if (ok && lane == 0 && t + WK_RING < total_tiles) issue(t + WK_RING);
    }
    while (cur < p.n_chunks) {  // leave the remaining chunks of this row block (also those this warp had no tile in)
      if (cur >= 0) leave_chunk(blk * p.n_chunks + cur);
      ++cur;
    }
    // ---- the four partial [16 x 32] sums meet in shared memory: red[warp][batch][row]
    {
      float* mine = red + warp * (WK_ROWS * SG_MAX_M);
      const int r0 = lane >> 2, bc = (lane & 3) * 2;
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        mine[(nt * 8 + bc) * WK_ROWS + r0] = acc[nt][0];
        mine[(nt * 8 + bc + 1) * WK_ROWS + r0] = acc[nt][1];
        mine[(nt * 8 + bc) * WK_ROWS + r0 + 8] = acc[nt][2];
        mine[(nt * 8 + bc + 1) * WK_ROWS + r0 + 8] = acc[nt][3];
      }
    }
    __syncthreads();
    {
      // thread -> batch row tid / 4, outputs (tid % 4) * 4 .. + 4: one 8-byte store
      const int b = tid >> 2, r = (tid & 3) * 4;
      float o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int idx = b * WK_ROWS + r + j;
        o[j] = ((red[idx] + red[WK_ROWS * SG_MAX_M + idx]) + red[2 * WK_ROWS * SG_MAX_M + idx]) +
               red[3 * WK_ROWS * SG_MAX_M + idx];
      }
      const int n0 = rb * WK_ROWS + r;
      if (b < p.m && n0 < p.n)  // N is a multiple of 8 and r of 4: the four outputs are inside or outside together
        *reinterpret_cast<uint2*>(p.y + static_cast<int64_t>(b) * p.y_stride + n0) =
            make_uint2(pack_bf16(o[0], o[1]), pack_bf16(o[2], o[3]));
    }
    __syncthreads();  // red is free for the next row block
  }
  if (!ok) {
    if (lane == 0) atomicExch(p.err, 1);
    // let this warp's copies in flight land before the shared memory goes away
    for (int s = 0; s < WK_RING; ++s) mbar_wait_bounded(&bars[warp][s], 0, 1u << 12);
    if (warp == 0) {
      mbar_wait_bounded(&bar_x[0], 0, 1u << 12);
      mbar_wait_bounded(&bar_x[1], 0, 1u << 12);
    }
  }
}

// ------------------------------------------------------------------------------------------------ pair-K form
// The same 16-outputs-per-step decomposition for K <= 4096, on a cluster of two CTAs that take one half of K each: twice
// as many SMs stream W, a CTA stages only its half of X -- once, whole, so there is no chunk pipeline -- and the two
// partial [16 x 32] sums meet through distributed shared memory (rank 1 stores its sum into rank 0's shared memory,
// one cluster barrier, rank 0 adds, rounds and writes).  No cluster multicast is used; every CTA loads its own tiles.
constexpr int PK_RING = 3;                 // W tiles in flight per warp (a warp has K / 1024 tiles per row block)
constexpr int PK_MAX_K = 4096;
constexpr int PK_SMEM = SG_WARPS * PK_RING * SG_TILE_BYTES + (SG_WARPS + 1) * WK_ROWS * SG_MAX_M * 4 +
                        SG_MAX_M * (PK_MAX_K + 16) + 1024;
static_assert(PK_SMEM <= 227 * 1024, "weight rings + half of X must fit the 227 KiB a CTA may use");

__global__ void __launch_bounds__(SG_THREADS, 1)
skinny_gemm_pairk_kernel(const __grid_constant__ WideKParams p, const __grid_constant__ CUtensorMap map_w) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ uint64_t bars[SG_WARPS][PK_RING];
  __shared__ uint64_t bar_x;
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t rank = cluster_ctarank();
  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
  uint8_t* ring = smem + warp * PK_RING * SG_TILE_BYTES;
  float* red = reinterpret_cast<float*>(smem + SG_WARPS * PK_RING * SG_TILE_BYTES);  // [4 warps + peer][32 batch][16 rows]
  float* peer = red + SG_WARPS * WK_ROWS * SG_MAX_M;                                 // written by rank 1 into rank 0
  uint8_t* xs = reinterpret_cast<uint8_t*>(peer + WK_ROWS * SG_MAX_M);               // [32][x_pitch]: this CTA's half of X
  const int half_k = p.k >> 1;
  const int x_pitch = half_k * 2 + 16;
  const int half_tiles = half_k / SG_TILE_K;

  if (tid == 0) {
    for (int w = 0; w < SG_WARPS; ++w)
      for (int s = 0; s < PK_RING; ++s) mbar_init(&bars[w][s], 1);
    mbar_init(&bar_x, 1);
    mbar_fence_init();
  }
  const int my_blocks = (p.row_blocks - pair + pairs - 1) / pairs;
  const int my_tiles = half_tiles > warp ? (half_tiles - warp + SG_WARPS - 1) / SG_WARPS : 0;  // per row block, this warp
  const int total_tiles = my_blocks * my_tiles;
  __syncthreads();
  auto issue = [&](int t) {  // lane 0: tile t of this warp
    const int rb = pair + (t / my_tiles) * pairs, kt = static_cast<int>(rank) * half_tiles + warp + SG_WARPS * (t % my_tiles);
    const int slot = t % PK_RING;
    mbar_expect_tx(&bars[warp][slot], SG_TILE_BYTES);
    tma_load_3d(ring + slot * SG_TILE_BYTES, &map_w, 0, rb * WK_ROWS, kt * 2, &bars[warp][slot]);
  };
  if (p.overlap & OVERLAP_TRIGGER) pdl_trigger();
  if (lane == 0) {
    for (int t = 0; t < PK_RING && t < total_tiles; ++t) issue(t);  // weights: independent of the predecessor
  }
  pdl_wait();  // X is the predecessor's output
  if (warp == 0) {
    if (lane == 0) mbar_expect_tx(&bar_x, static_cast<uint32_t>(p.m) * half_k * 2);
    __syncwarp();
    if (lane < p.m)
      bulk_g2s(xs + lane * x_pitch, p.x + static_cast<int64_t>(lane) * p.x_stride + rank * half_k, half_k * 2, &bar_x);
  }
  for (int i = tid; i < (SG_MAX_M - p.m) * (half_k >> 3); i += SG_THREADS) {  // rows beyond M are zero
    const int r = p.m + i / (half_k >> 3), c = i % (half_k >> 3);
    *reinterpret_cast<uint4*>(xs + r * x_pitch + c * 16) = make_uint4(0, 0, 0, 0);
  }
  __syncthreads();
  bool ok = mbar_wait_bounded(&bar_x, 0);

  const int a_row = lane & 15, a_par = lane >> 4;
  const uint32_t xs_base = smem_u32(xs) + static_cast<uint32_t>(((lane & 7) + ((lane >> 4) << 3)) * x_pitch + ((lane >> 3) & 1) * 16);
  const uint32_t peer_remote = cluster_map(smem_u32(peer), 0);
  int t = 0;
  for (int blk = 0; blk < my_blocks; ++blk) {
    const int rb = pair + blk * pairs;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
    for (int kl = warp; kl < half_tiles; kl += SG_WARPS, ++t) {
      const int slot = t % PK_RING;
      if (ok && !mbar_wait_bounded(&bars[warp][slot], (t / PK_RING) & 1)) ok = false;
      if (ok) {
        const uint32_t tile = smem_u32(ring + slot * SG_TILE_BYTES);
        const uint32_t xk0 = xs_base + kl * SG_TILE_K * 2;
#pragma unroll
        for (int ks = 0; ks < SG_TILE_K / 16; ++ks) {
          uint32_t a[4], b01[4], b23[4];
          const uint32_t a_off = (ks >> 2) * (16 * 128) + a_row * 128 + ((((ks & 3) * 2 + a_par) ^ (a_row & 7)) << 4);
          ldmatrix_x4(b01, xk0 + ks * 32);
          ldmatrix_x4(b23, xk0 + ks * 32 + 16 * x_pitch);
          ldmatrix_x4(a, tile + a_off);
          mma_bf16_16816(acc[0], a, b01[0], b01[1]);
          mma_bf16_16816(acc[1], a, b01[2], b01[3]);
          mma_bf16_16816(acc[2], a, b23[0], b23[1]);
          mma_bf16_16816(acc[3], a, b23[2], b23[3]);
        }
      }
      __syncwarp();  // every lane has read the tile: its slot can take the tile PK_RING ahead
      if (ok && lane == 0 && t + PK_RING < total_tiles) issue(t + PK_RING);
    }
    // ---- the warps' partial [16 x 32] sums meet in shared memory: red[warp][batch][row]
    {
      float* mine = red + warp * (WK_ROWS * SG_MAX_M);
      const int r0 = lane >> 2, bc = (lane & 3) * 2;
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        mine[(nt * 8 + bc) * WK_ROWS + r0] = acc[nt][0];
        mine[(nt * 8 + bc + 1) * WK_ROWS + r0] = acc[nt][1];
        mine[(nt * 8 + bc) * WK_ROWS + r0 + 8] = acc[nt][2];
        mine[(nt * 8 + bc + 1) * WK_ROWS + r0 + 8] = acc[nt][3];
      }
    }
    __syncthreads();
    // thread -> batch row tid / 4, outputs (tid % 4) * 4 .. + 4
    const int b = tid >> 2, r = (tid & 3) * 4;
    float o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int idx = b * WK_ROWS + r + j;
      o[j] = ((red[idx] + red[WK_ROWS * SG_MAX_M + idx]) + red[2 * WK_ROWS * SG_MAX_M + idx]) +
             red[3 * WK_ROWS * SG_MAX_M + idx];
    }
    if (rank == 1) st_cluster_f32x4(peer_remote + (b * WK_ROWS + r) * 4, o[0], o[1], o[2], o[3]);
    cluster_sync();  // rank 1's sum is in rank 0's shared memory; red is free again in both CTAs
    if (rank == 0) {
      const float4 other = *reinterpret_cast<const float4*>(peer + b * WK_ROWS + r);
      const int n0 = rb * WK_ROWS + r;
      if (b < p.m && n0 < p.n)  // N is a multiple of 8 and r of 4: the four outputs are inside or outside together
        *reinterpret_cast<uint2*>(p.y + static_cast<int64_t>(b) * p.y_stride + n0) =
            make_uint2(pack_bf16(o[0] + other.x, o[1] + other.y), pack_bf16(o[2] + other.z, o[3] + other.w));
    }
    if (blk + 1 < my_blocks) cluster_sync();  // rank 0 has read `peer` before rank 1 writes the next sum
  }
  if (!ok) {
    if (lane == 0) atomicExch(p.err, 1);
    // let this warp's copies in flight land before the shared memory goes away
    for (int s = 0; s < PK_RING; ++s) mbar_wait_bounded(&bars[warp][s], 0, 1u << 12);
    if (warp == 0) mbar_wait_bounded(&bar_x, 0, 1u << 12);
  }
}

// Shared by all host threads: searched and filled under a mutex, the map is copied out.
static bool cache_weight_map(const void* base, int64_t n, int64_t k, int box_rows, CUtensorMap* out) {
  static std::mutex mu;
  std::lock_guard<std::mutex> lock(mu);
  struct Entry {
    const void* base;
    int64_t n, k;
    int dev, box_rows;
    CUtensorMap map;
  };
  constexpr int N = 128;  // a model has a fixed set of weight matrices
  static Entry entries[N];
  static int used = 0, next = 0;
  int dev = 0;
  cudaGetDevice(&dev);
  for (int i = 0; i < used; ++i)
    if (entries[i].base == base && entries[i].n == n && entries[i].k == k && entries[i].dev == dev &&
        entries[i].box_rows == box_rows) {
      *out = entries[i].map;
      return true;
    }
  Entry& e = entries[next];
  e.base = nullptr;  // not a valid entry while it is being rewritten
  if (!encode_tile_map(&e.map, base, static_cast<uint64_t>(n), static_cast<uint64_t>(k), static_cast<uint64_t>(k) * 2, box_rows, 2))
    return false;
  e.base = base;
  e.n = n;
  e.k = k;
  e.dev = dev;
  e.box_rows = box_rows;
  next = (next + 1) % N;
  if (used < N) ++used;
  *out = e.map;
  return true;
}

}  // namespace b200

using namespace b200;

template <bool SWIGLU, bool ARGMAX = false>
static int launch_skinny(SkinnyGemmParams p, const void* weight, int w_rows, cudaStream_t stream, const char* what) {
  CUtensorMap map;
  if (!cache_weight_map(weight, w_rows, p.k, SWIGLU ? 8 : 16, &map)) return fail(ERR_RUNTIME, "%s: cannot encode the weight tensor map", what);
  constexpr int smem_max =
      SG_WARPS * SG_RING_BYTES + SG_MAX_M * SG_ROWS * 2 + SG_PART_BYTES + SG_MAX_M * (SG_MAX_K * 2 + 16) + 1024;
  static_assert(smem_max <= 227 * 1024, "weight rings + X staging must fit the 227 KiB a CTA may use");
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    if (cudaFuncSetAttribute(skinny_gemm_kernel<SWIGLU, ARGMAX>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_max) !=
        cudaSuccess)
      return fail(ERR_RUNTIME, "%s: cannot raise dynamic shared memory to %d", what, smem_max);
    configured[dev] = true;
  }
  p.err = wait_timeout_flag();
  if (!p.err) return fail(ERR_RUNTIME, "%s: no error flag", what);
  constexpr int out_per_cta = SWIGLU ? 8 * SG_WARPS : SG_ROWS;
  p.row_blocks = (p.n + out_per_cta - 1) / out_per_cta;
  int grid = p.row_blocks;
  const int sms = sm_count();
  if (grid > sms) grid = sms;
  const int dyn = SG_WARPS * SG_RING_BYTES + SG_MAX_M * SG_ROWS * 2 + SG_PART_BYTES + SG_MAX_M * (p.k * 2 + 16) + 1024;
  if (launch_pdl((p.overlap & OVERLAP_START) != 0, skinny_gemm_kernel<SWIGLU, ARGMAX>, dim3(grid), dim3(SG_STD_THREADS), dyn, stream,
                 p, map) != cudaSuccess)
    return fail(ERR_LAUNCH, "%s: %s", what, cudaGetErrorString(cudaGetLastError()));
  return check_launch(what);
}

// Chunking of K for the wide-K form: the fewest equal chunks of whole 128-k tiles that are at most WK_CHUNK_MAX long.
static bool widek_chunks(int k, int* chunk_k, int* n_chunks) {
  if (k <= 0 || k % SG_TILE_K != 0 || k > WK_MAX_K) return false;
  const int n = (k + WK_CHUNK_MAX - 1) / WK_CHUNK_MAX;
  if (k % (n * SG_TILE_K) != 0) return false;
  *chunk_k = k / n;
  *n_chunks = n;
  return true;
}

static int launch_widek(WideKParams p, const void* weight, cudaStream_t stream) {
  const char* what = "skinny_gemm";
  CUtensorMap map;
  if (!cache_weight_map(weight, p.n, p.k, 16, &map)) return fail(ERR_RUNTIME, "%s: cannot encode the weight tensor map", what);
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    if (cudaFuncSetAttribute(skinny_gemm_widek_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, WK_SMEM) != cudaSuccess)
      return fail(ERR_RUNTIME, "%s: cannot raise dynamic shared memory to %d", what, WK_SMEM);
    configured[dev] = true;
  }
  p.err = wait_timeout_flag();
  if (!p.err) return fail(ERR_RUNTIME, "%s: no error flag", what);
  p.row_blocks = (p.n + WK_ROWS - 1) / WK_ROWS;
  int grid = p.row_blocks;
  const int sms = sm_count();
  if (grid > sms) grid = sms;
  const int dyn = SG_WARPS * WK_RING * SG_TILE_BYTES + SG_WARPS * WK_ROWS * SG_MAX_M * 4 +
                  2 * SG_MAX_M * (p.chunk_k * 2 + 16) + 1024;
  if (launch_pdl((p.overlap & OVERLAP_START) != 0, skinny_gemm_widek_kernel, dim3(grid), dim3(SG_THREADS), dyn, stream, p,
                 map) != cudaSuccess)
    return fail(ERR_LAUNCH, "%s: %s", what, cudaGetErrorString(cudaGetLastError()));
  return check_launch(what);
}

static int launch_pairk(WideKParams p, const void* weight, cudaStream_t stream) {
  const char* what = "skinny_gemm";
  CUtensorMap map;
  if (!cache_weight_map(weight, p.n, p.k, 16, &map)) return fail(ERR_RUNTIME, "%s: cannot encode the weight tensor map", what);
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    if (cudaFuncSetAttribute(skinny_gemm_pairk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PK_SMEM) != cudaSuccess)
      return fail(ERR_RUNTIME, "%s: cannot raise dynamic shared memory to %d", what, PK_SMEM);
    configured[dev] = true;
  }
  p.err = wait_timeout_flag();
  if (!p.err) return fail(ERR_RUNTIME, "%s: no error flag", what);
  p.row_blocks = (p.n + WK_ROWS - 1) / WK_ROWS;
  int pairs = p.row_blocks;
  const int sms = sm_count();
  if (pairs > sms / 2) pairs = sms / 2;
  const int dyn = SG_WARPS * PK_RING * SG_TILE_BYTES + (SG_WARPS + 1) * WK_ROWS * SG_MAX_M * 4 +
                  SG_MAX_M * (p.k + 16) + 1024;
  if (launch_pdl_cluster((p.overlap & OVERLAP_START) != 0, 2, skinny_gemm_pairk_kernel, dim3(2 * pairs), dim3(SG_THREADS),
                         dyn, stream, p, map) != cudaSuccess)
    return fail(ERR_LAUNCH, "%s: %s", what, cudaGetErrorString(cudaGetLastError()));
  return check_launch(what);
}

static int check_skinny_shape(const char* what, int m, int n, int k) {
  B200_REQUIRE(m > 0 && m <= SG_MAX_M, "%s: M must be in [1, %d] (got %d)", what, SG_MAX_M, m);
  B200_REQUIRE(n > 0 && n % 8 == 0 && k >= SG_TILE_K && k % SG_TILE_K == 0 && k <= SG_MAX_K,
               "%s: N must be a multiple of 8, K a multiple of %d up to %d (got N=%d K=%d)", what, SG_TILE_K, SG_MAX_K, n,
               k);
  return OK;
}

extern "C" int b200_skinny_gemm(const void* x, int64_t x_stride, const void* weight, void* y, int64_t y_stride,
                                int32_t m, int32_t n, int32_t k, int32_t overlap, b200_stream_t stream) {
  B200_REQUIRE(aligned16(x) && aligned16(weight) && aligned16(y) && x_stride % 8 == 0 && y_stride % 8 == 0,
               "skinny_gemm: pointers must be 16-byte aligned, row strides multiples of 8 elements");
  if (k > SG_MAX_K) {  // long rows: K split over the warps of a CTA, X staged in chunks
    WideKParams wp = {};
    B200_REQUIRE(m > 0 && m <= SG_MAX_M && n > 0 && n % 8 == 0 && widek_chunks(k, &wp.chunk_k, &wp.n_chunks),
                 "skinny_gemm: M must be in [1, %d], N a multiple of 8, K > %d a multiple of 128 that splits into equal "
                 "chunks of whole tiles of at most %d (got M=%d N=%d K=%d)", SG_MAX_M, SG_MAX_K, WK_CHUNK_MAX, m, n, k);
    wp.x = static_cast<const __nv_bfloat16*>(x);
    wp.y = static_cast<__nv_bfloat16*>(y);
    wp.x_stride = x_stride;
    wp.y_stride = y_stride;
    wp.m = m;
    wp.n = n;
    wp.k = k;
    wp.overlap = overlap;
    if (k <= PK_MAX_K && k % (2 * SG_TILE_K) == 0) return launch_pairk(wp, weight, reinterpret_cast<cudaStream_t>(stream));
    return launch_widek(wp, weight, reinterpret_cast<cudaStream_t>(stream));
  }
  int rc = check_skinny_shape("skinny_gemm", m, n, k);
  if (rc != OK) return rc;
  SkinnyGemmParams p = {};
  p.x = static_cast<const __nv_bfloat16*>(x);
  p.y = static_cast<__nv_bfloat16*>(y);
  p.x_stride = x_stride;
  p.y_stride = y_stride;
  p.m = m;
  p.n = n;
  p.k = k;
  p.overlap = overlap;
  return launch_skinny<false>(p, weight, n, reinterpret_cast<cudaStream_t>(stream), "skinny_gemm");
}

extern "C" int b200_skinny_gemm_swiglu(const void* x, int64_t x_stride, const void* weight, void* y, int64_t y_stride,
                                       int32_t m, int32_t intermediate, int32_t k, int32_t overlap,
                                       b200_stream_t stream) {
  int rc = check_skinny_shape("skinny_gemm_swiglu", m, intermediate, k);
  if (rc != OK) return rc;
  B200_REQUIRE(aligned16(x) && aligned16(weight) && aligned16(y) && x_stride % 8 == 0 && y_stride % 8 == 0,
               "skinny_gemm_swiglu: pointers must be 16-byte aligned, row strides multiples of 8 elements");
  SkinnyGemmParams p = {};
  p.x = static_cast<const __nv_bfloat16*>(x);
  p.y = static_cast<__nv_bfloat16*>(y);
  p.x_stride = x_stride;
  p.y_stride = y_stride;
  p.m = m;
  p.n = intermediate;
  p.k = k;
  p.overlap = overlap;
  p.up_row0 = intermediate;
  return launch_skinny<true>(p, weight, 2 * intermediate, reinterpret_cast<cudaStream_t>(stream), "skinny_gemm_swiglu");
}

extern "C" int b200_lm_head_argmax(const void* x, int64_t x_stride, const void* weight, int64_t* ids, void* workspace,
                                   int32_t m, int32_t n, int32_t k, int32_t overlap, b200_stream_t stream) {
  int rc = check_skinny_shape("lm_head_argmax", m, n, k);
  if (rc != OK) return rc;
  B200_REQUIRE(aligned16(x) && aligned16(weight) && x_stride % 8 == 0 && ids != nullptr && workspace != nullptr &&
                   (reinterpret_cast<uintptr_t>(workspace) % 8 == 0),
               "lm_head_argmax: x / weight must be 16-byte aligned, the x row stride a multiple of 8, the workspace "
               "8-byte aligned");
  SkinnyGemmParams p = {};
  p.x = static_cast<const __nv_bfloat16*>(x);
  p.x_stride = x_stride;
  p.m = m;
  p.n = n;
  p.k = k;
  p.overlap = overlap;
  p.ids = ids;
  p.keys = static_cast<unsigned long long*>(workspace);  // the layout of b200_argmax_rows: 1024 keys, then counters
  p.counter = reinterpret_cast<int*>(p.keys + 1024);
  return launch_skinny<false, true>(p, weight, n, reinterpret_cast<cudaStream_t>(stream), "lm_head_argmax");
}
