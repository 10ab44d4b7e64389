// Reference-compatible split-K pair for paged GQA decode attention:
//   b200_paged_decode_split   <->  triton_kernels/gqa_attention_decode_paged.py:622-733 (+ op :822-891)
//   b200_paged_decode_combine <->  triton_kernels/gqa_attention_decode_paged.py:745-817 (+ op :901-939)
// The page partition (pages_per_split = cdiv(pages_used, 128), split s owns pages
// [s*pps, min((s+1)*pps, pages_used))) and the scratch layout are the reference's, so either half can be
// mixed with the reference's other half.  All 128 partials are written, empty ones as (-inf, 0, 0).
#include "b200_attn.h"
#include "decode_core.cuh"

namespace b200 {

constexpr int SPLIT_WARPS = 4;
constexpr int SPLIT_TILES = 2;  // K and V tile of one page per warp: 66 KiB per CTA, three CTAs (12 warps) per SM.  With the
                                // reference's partition a warp owns one or two pages and writes a 4 KiB partial, so
                                // the launch is bound by per-item latency: resident warps matter more than a deep ring
constexpr int SPLIT_TILES_DEEP = 4;  // launches of at most one CTA per SM (one or two sequences): both pages of a warp's
                                     // split are requested at once instead of the second behind the first
constexpr int split_smem(int tiles) { return SPLIT_WARPS * tiles * TILE_BYTES + 128; }

// One warp per (sequence, kv head, split).  grid.x = B * H_kv * 128 / SPLIT_WARPS: static in B, so the launch
// is CUDA-graph safe; everything length-dependent comes from pos[] on the device.
template <int TILES>
__global__ void __launch_bounds__(SPLIT_WARPS * 32, TILES == SPLIT_TILES ? 3 : 1)
paged_decode_split_kernel(const __nv_bfloat16* q, int64_t q_b, int64_t q_h,
                          const __nv_bfloat16* k_cache, const __nv_bfloat16* v_cache,
                          int64_t kc_p, int64_t kc_h, int64_t kc_s, int64_t vc_p, int64_t vc_h, int64_t vc_s,
                          const int32_t* block_table, int64_t bt_b, float* m_partial,
                          float* l_partial, float* acc_partial,
                          const int64_t* pos, int num_kv_heads, float scale, int* err) {
  pdl_chain();
  extern __shared__ __align__(128) uint8_t smem_raw[];
  __shared__ uint64_t bars[SPLIT_WARPS][TILES];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
  uint8_t* ring = smem + warp * TILES * TILE_BYTES;
  if (lane == 0) {
    for (int s = 0; s < TILES; ++s) mbar_init(&bars[warp][s], 1);
    mbar_fence_init();
  }
  __syncwarp();

  const int item = blockIdx.x * SPLIT_WARPS + warp;
  const int split = item % MAX_SPLITS;
  const int h = (item / MAX_SPLITS) % num_kv_heads;
  const int b = item / (MAX_SPLITS * num_kv_heads);
  const int num_q_heads = num_kv_heads * GROUP;

  const int seq_len = static_cast<int>(pos[b]) + 1;
  const int pages_used = (seq_len + PAGE - 1) / PAGE;
  const int pps = (pages_used + MAX_SPLITS - 1) / MAX_SPLITS;
  const int page_start = split * pps;
  const int page_end = min(page_start + pps, pages_used);
  const int n_pages = max(page_end - page_start, 0);

  DecodeWarpState st;
  decode_state_init(st);
  const int32_t* table = block_table + b * bt_b;
  const __nv_bfloat16* kh = k_cache + h * kc_h;
  const __nv_bfloat16* vh = v_cache + h * vc_h;

  if (n_pages > 0) {
    decode_load_q(st, q + b * q_b + (h * GROUP) * q_h, q_h, lane);
    // tile t = K (even) or V (odd) of page t/2, staged in ring slot t % TILES
    auto issue = [&](int t) {
      const int64_t phys = table[page_start + (t >> 1)];
      const int slot = t % TILES;
      if (t & 1) decode_issue_tile(ring + slot * TILE_BYTES, &bars[warp][slot], vh + phys * vc_p, vc_s, lane);
      else decode_issue_tile(ring + slot * TILE_BYTES, &bars[warp][slot], kh + phys * kc_p, kc_s, lane);
    };
    const int n_tiles = 2 * n_pages;
    for (int t = 0; t < min(n_tiles, TILES); ++t) issue(t);
    bool ok = true;
    for (int i = 0; i < n_pages && ok; ++i) {
      const int valid = min(PAGE, seq_len - (page_start + i) * PAGE);
      uint32_t b0 = 0, b1 = 0;
      float alpha0 = 1.f, alpha1 = 1.f;
#pragma unroll
      for (int part = 0; part < 2; ++part) {
        const int t = 2 * i + part;
        const int slot = t % TILES;
        if (!mbar_wait_bounded(&bars[warp][slot], (t / TILES) & 1)) {
          ok = false;
          break;
        }
        uint8_t* tile = ring + slot * TILE_BYTES;
        if (part == 0) decode_scores(st, tile, valid, scale, lane, b0, b1, alpha0, alpha1);
        else decode_accumulate(st, tile, valid, b0, b1, alpha0, alpha1, lane);
        fence_proxy_async();  // row clears (generic proxy) before the next bulk copy into this slot
        __syncwarp();
        if (t + TILES < n_tiles) issue(t + TILES);
      }
    }
    if (!ok) {
      if (lane == 0) atomicExch(err, 1);
      // copies may still be in flight into this CTA's shared memory: give them a bounded time to land
      for (int s = 0; s < TILES; ++s) mbar_wait_bounded(&bars[warp][s], 0, 1u << 12);
      return;
    }
    decode_reduce_l(st);
  }

  // ---- store the partial: m, l per head; acc through shared memory for 16-byte coalesced stores
  const int hq0 = h * GROUP;
  if (lane < 2) {
    const int64_t base = (static_cast<int64_t>(b) * num_q_heads + hq0 + lane * 2) * MAX_SPLITS + split;
    m_partial[base] = st.m[0];
    m_partial[base + MAX_SPLITS] = st.m[1];
    l_partial[base] = st.l[0];
    l_partial[base + MAX_SPLITS] = st.l[1];
  }
  float* tile = reinterpret_cast<float*>(ring);
  __syncwarp();
  decode_store_acc_smem(st, tile, lane);
  __syncwarp();
#pragma unroll
  for (int j = 0; j < GROUP * HEAD_DIM / 4 / 32; ++j) {
    const int idx = j * 32 + lane;  // float4 index inside the [4][256] tile
    const int head = idx / (HEAD_DIM / 4), c = idx % (HEAD_DIM / 4);
    float4 v = reinterpret_cast<const float4*>(tile)[idx];
    float* dst = acc_partial + ((static_cast<int64_t>(b) * num_q_heads + hq0 + head) * MAX_SPLITS + split) * HEAD_DIM;
    reinterpret_cast<float4*>(dst)[c] = v;
  }
}

// One CTA per (sequence, q head).  Thread t takes 4 output dims (t % 64) of the splits s = t / 64, + 4, + 8, ...: 16-byte
// loads, a quarter of the splits deep, sixteen loads in flight per thread; the four groups meet in shared memory and are
// added in a fixed order.  Every warp forms the global max and the rescaled sum of l for itself (4 values of m and l per
// lane), so the only barrier is the one in front of the final sum.
__global__ void __launch_bounds__(HEAD_DIM)
paged_decode_combine_kernel(const float* m_partial, const float* l_partial,
                            const float* acc_partial, const int64_t* pos,
                            __nv_bfloat16* out, int num_q_heads) {
  pdl_chain();
  static_assert(MAX_SPLITS == 128 && HEAD_DIM == 256, "the lane / group mapping below is written for 128 splits x 256 dims");
  const int b = blockIdx.x, hq = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int c = tid & 63, sg = tid >> 6;
  const int seq_len = static_cast<int>(pos[b]) + 1;
  const int pages_used = (seq_len + PAGE - 1) / PAGE;
  const int pps = (pages_used + MAX_SPLITS - 1) / MAX_SPLITS;
  const int num_active = (pages_used + pps - 1) / pps;
  const int64_t row = static_cast<int64_t>(b) * num_q_heads + hq;
  const float* m = m_partial + row * MAX_SPLITS;
  const float* l = l_partial + row * MAX_SPLITS;
  const float4* acc = reinterpret_cast<const float4*>(acc_partial + row * MAX_SPLITS * HEAD_DIM) + c;
  __shared__ float alpha_s[HEAD_DIM / 32][MAX_SPLITS];
  __shared__ float4 part[4][HEAD_DIM / 4];
  float mv[4], lv[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int s = lane + 32 * i;
    mv[i] = s < num_active ? m[s] : -INFINITY;
    lv[i] = s < num_active ? l[s] : 0.f;
  }
  // the first sixteen accumulator rows of this thread are requested together with m and l: one round trip, not two
  float4 x[16];
#pragma unroll
  for (int u = 0; u < 16; ++u) {
    const int s = sg + 4 * u;
    x[u] = s < num_active ? acc[static_cast<int64_t>(s) * (HEAD_DIM / 4)] : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  const float mx = warp_max(fmaxf(fmaxf(mv[0], mv[1]), fmaxf(mv[2], mv[3])));
  float lsum = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float a = (mv[i] == -INFINITY) ? 0.f : __expf(mv[i] - mx);  // an empty split weighs nothing
    alpha_s[warp][lane + 32 * i] = a;
    lsum += lv[i] * a;
  }
  lsum = warp_sum(lsum);
  __syncwarp();
  float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int s0 = sg; s0 < num_active; s0 += 64) {
    if (s0 != sg) {
#pragma unroll
      for (int u = 0; u < 16; ++u) {
        const int s = s0 + 4 * u;
        x[u] = s < num_active ? acc[static_cast<int64_t>(s) * (HEAD_DIM / 4)] : make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
#pragma unroll
    for (int u = 0; u < 16; ++u) {
      const int s = s0 + 4 * u;
      const float a = s < num_active ? alpha_s[warp][s] : 0.f;
      sum.x = fmaf(x[u].x, a, sum.x);
      sum.y = fmaf(x[u].y, a, sum.y);
      sum.z = fmaf(x[u].z, a, sum.z);
      sum.w = fmaf(x[u].w, a, sum.w);
    }
  }
  part[sg][c] = sum;
  __syncthreads();
  if (sg == 0) {
    const float4 p1 = part[1][c], p2 = part[2][c], p3 = part[3][c];
    const float o0 = ((sum.x + p1.x) + (p2.x + p3.x)) / lsum, o1 = ((sum.y + p1.y) + (p2.y + p3.y)) / lsum;
    const float o2 = ((sum.z + p1.z) + (p2.z + p3.z)) / lsum, o3 = ((sum.w + p1.w) + (p2.w + p3.w)) / lsum;
    *reinterpret_cast<uint2*>(out + row * HEAD_DIM + c * 4) = make_uint2(pack_bf16(o0, o1), pack_bf16(o2, o3));
  }
}

}  // namespace b200

using namespace b200;

extern "C" int b200_paged_decode_split(const void* q, int64_t q_stride_b, int64_t q_stride_h, const void* k_cache,
                                       const void* v_cache, int64_t kc_stride_p, int64_t kc_stride_h,
                                       int64_t kc_stride_s, int64_t vc_stride_p, int64_t vc_stride_h,
                                       int64_t vc_stride_s, const int32_t* block_table, int64_t bt_stride_b,
                                       float* m_partial, float* l_partial, float* acc_partial, const int64_t* pos,
                                       int32_t batch, int32_t num_q_heads, int32_t num_kv_heads, int32_t head_dim,
                                       b200_stream_t stream) {
  B200_REQUIRE(batch > 0, "paged_decode_split: batch must be positive");
  B200_REQUIRE(head_dim == HEAD_DIM, "paged_decode_split: head_dim must be %d (got %d)", HEAD_DIM, head_dim);
  B200_REQUIRE(num_kv_heads > 0 && num_q_heads == num_kv_heads * GROUP,
               "paged_decode_split: needs %d Q heads per KV head (got %d/%d)", GROUP, num_q_heads, num_kv_heads);
  B200_REQUIRE(aligned16(k_cache) && aligned16(v_cache) && aligned16(acc_partial) && (kc_stride_s % 8 == 0) &&
                   (vc_stride_s % 8 == 0) && (kc_stride_p % 8 == 0) && (vc_stride_p % 8 == 0) &&
                   (kc_stride_h % 8 == 0) && (vc_stride_h % 8 == 0),
               "paged_decode_split: caches and scratch must be 16-byte aligned with strides that are multiples of 8");
  B200_REQUIRE((reinterpret_cast<uintptr_t>(q) % 4 == 0) && (q_stride_b % 2 == 0) && (q_stride_h % 2 == 0),
               "paged_decode_split: q must be 4-byte aligned with even strides");
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    if (cudaFuncSetAttribute(paged_decode_split_kernel<SPLIT_TILES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             split_smem(SPLIT_TILES)) != cudaSuccess ||
        cudaFuncSetAttribute(paged_decode_split_kernel<SPLIT_TILES_DEEP>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             split_smem(SPLIT_TILES_DEEP)) != cudaSuccess)
      return fail(ERR_RUNTIME, "paged_decode_split: cannot raise dynamic shared memory to %d", split_smem(SPLIT_TILES_DEEP));
    configured[dev] = true;
  }
  int* err = wait_timeout_flag();
  if (!err) return fail(ERR_RUNTIME, "paged_decode_split: no error flag");
  const int64_t items = static_cast<int64_t>(batch) * num_kv_heads * MAX_SPLITS;
  const unsigned grid = static_cast<unsigned>(items / SPLIT_WARPS);
  if (static_cast<int>(grid) <= sm_count())
    launch_pdl(chain_overlap(), paged_decode_split_kernel<SPLIT_TILES_DEEP>, dim3(grid), dim3(SPLIT_WARPS * 32), split_smem(SPLIT_TILES_DEEP), reinterpret_cast<cudaStream_t>(stream),
             
        static_cast<const __nv_bfloat16*>(q), q_stride_b, q_stride_h, static_cast<const __nv_bfloat16*>(k_cache),
        static_cast<const __nv_bfloat16*>(v_cache), kc_stride_p, kc_stride_h, kc_stride_s, vc_stride_p, vc_stride_h,
        vc_stride_s, block_table, bt_stride_b, m_partial, l_partial, acc_partial, pos, num_kv_heads,
        1.0f / sqrtf(static_cast<float>(head_dim)), err);
  else
    launch_pdl(chain_overlap(), paged_decode_split_kernel<SPLIT_TILES>, dim3(grid), dim3(SPLIT_WARPS * 32), split_smem(SPLIT_TILES), reinterpret_cast<cudaStream_t>(stream),
             
        static_cast<const __nv_bfloat16*>(q), q_stride_b, q_stride_h, static_cast<const __nv_bfloat16*>(k_cache),
        static_cast<const __nv_bfloat16*>(v_cache), kc_stride_p, kc_stride_h, kc_stride_s, vc_stride_p, vc_stride_h,
        vc_stride_s, block_table, bt_stride_b, m_partial, l_partial, acc_partial, pos, num_kv_heads,
        1.0f / sqrtf(static_cast<float>(head_dim)), err);
  return check_launch("paged_decode_split");
}

extern "C" int b200_paged_decode_combine(const float* m_partial, const float* l_partial, const float* acc_partial,
                                         const int64_t* pos, void* out, int32_t batch, int32_t num_q_heads,
                                         int32_t head_dim, b200_stream_t stream) {
  B200_REQUIRE(batch > 0 && num_q_heads > 0 && num_q_heads <= 65535, "paged_decode_combine: bad shape");
  B200_REQUIRE(head_dim == HEAD_DIM, "paged_decode_combine: head_dim must be %d (got %d)", HEAD_DIM, head_dim);
  launch_pdl(chain_overlap(), paged_decode_combine_kernel, dim3(batch, num_q_heads), dim3(HEAD_DIM), 0, reinterpret_cast<cudaStream_t>(stream),
             
      m_partial, l_partial, acc_partial, pos, static_cast<__nv_bfloat16*>(out), num_q_heads);
  return check_launch("paged_decode_combine");
}

