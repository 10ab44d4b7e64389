// Fused paged GQA decode attention for one layer step:
//   partial RoPE(q, k_new) at pos[b]  ->  append(k_new, v_new)  ->  attention over pos[b]+1 tokens  ->  sigmoid gate
// in ONE launch.  It replaces the operator chain of engine/runner.py:482-517 in the reference
// (partial_rope x2, paged_kv_append, paged_gqa_attention_decode_split, ..._combine, attention_gate_pack; the
// attention part is call_paged_gqa_attention_decode_triton, triton_kernels/gqa_attention_decode_paged.py:963-994).
//
// Work decomposition ("stream-K over pages").  A unit is one KV page of one (sequence, kv head) segment, plus
// one extra unit per segment for the token being appended.  All units of all segments form one line (with a gap
// behind every segment that stands for the cost of stopping at a segment boundary, see Segment) that is
// cut into equal ranges, one per CTA; the grid is one CTA per SM whatever the batch or the context lengths,
// and the cut is recomputed on the device from pos[], so the launch is static and CUDA-graph safe.  Inside a
// CTA the eight warps take the units of a segment piece round-robin, each with a private ring of three
// K/V tiles, each tile filled by ONE tensor-map TMA copy (8 KiB box, 128-byte swizzle; decode_core.cuh), then merge
// their online-softmax states through shared memory.
//   - A segment that lies inside one CTA's range is finished there: normalise, round to bf16, multiply by
//     sigmoid(gate), store.
//   - A segment cut by a range boundary leaves one partial (m, l, acc[4][256]) per CTA in the workspace; the
//     last CTA to arrive (a counter per segment) merges them and finishes the segment.  No CTA ever waits for
//     another one, so nothing depends on co-residency.
// Small batches (up to 64 segments) are launched as thread-block clusters and may give each SEGMENT to one cluster
// instead: its CTAs split the segment's pages evenly, exchange their online-softmax states through distributed shared
// memory - every CTA receives one slice of the output dims from all the others, so the exchange is 4 KiB per CTA
// whatever the cluster size - meet at one cluster barrier and finish their slice.  No global partials, tickets or
// fences, and no CTA streams more than 1/cluster of the longest segment.
// The appended token never takes the cross-CTA write-then-read path that makes the reference keep the append
// in its own launch (gqa_attention_decode_paged.py:332-334): its K/V rows are built in shared memory by the warp
// that owns the segment's extra unit and stored to the cache from there; page readers mask that slot.
#include "b200_attn.h"
#include "decode_core.cuh"
#include "umma.cuh"

#include <mutex>

namespace b200 {

constexpr int FD_WARPS = 8;
constexpr int FD_THREADS = FD_WARPS * 32;
constexpr int FD_RING = 3;                             // K/V tiles per warp
constexpr int FD_MERGE_SLOTS = 4;                      // warps merge in two rounds of four
constexpr int FD_MAX_BATCH = 512;                      // prefix table and positions live in shared memory
constexpr int FD_MAX_SEGMENTS = 2048;                  // counters in the workspace
constexpr int FD_MAX_CTAS = 256;                       // partial slots in the workspace
constexpr int FD_TILE_FLOATS = GROUP * HEAD_DIM;       // 1024 accumulator floats per partial
constexpr int FD_PARTIAL_FLOATS = FD_TILE_FLOATS + 8;  // + m[4], l[4]
constexpr int64_t FD_COUNTER_BYTES = FD_MAX_SEGMENTS * 4;
constexpr int64_t FD_WORKSPACE_BYTES = FD_COUNTER_BYTES + int64_t(FD_MAX_CTAS) * 2 * FD_PARTIAL_FLOATS * 4;

constexpr int FD_SMEM_RING = FD_WARPS * FD_RING * TILE_BYTES_SW;
constexpr int FD_SMEM_MERGE = FD_MERGE_SLOTS * FD_PARTIAL_FLOATS * 4;
constexpr int FD_SMEM_CUM = ((FD_MAX_BATCH + 1) * 4 + 15) / 16 * 16;   // exclusive prefix of units
constexpr int FD_SMEM_POS = FD_MAX_BATCH * 4;                           // pos[] as int32
constexpr int FD_Q_PITCH = HEAD_DIM + 8;                                // bf16 elements per staged Q row
constexpr int FD_SMEM_Q = 2 * GROUP * FD_Q_PITCH * 2;                   // rotated Q of this piece and of the next
constexpr int FD_GAP = 32;                                              // line positions behind every segment (see Segment)
constexpr int FD_MAX_CLUSTER = 16;                                      // CTAs that may share one segment
constexpr int FD_SMEM_RECV = FD_TILE_FLOATS * 4 + FD_MAX_CLUSTER * 8 * 4;  // cluster exchange: one accumulator slice per
                                                                           // source CTA (4 KiB in all) + every (m, l)
constexpr int FD_SMEM_TOTAL =
    FD_SMEM_RING + FD_SMEM_MERGE + FD_SMEM_CUM + FD_SMEM_POS + FD_SMEM_Q + FD_SMEM_RECV + 1024;
static_assert(FD_SMEM_TOTAL <= 227 * 1024, "shared memory budget");

struct FusedDecodeParams {
  int gap;  // empty positions behind every segment on the unit line (see Segment)
  const __nv_bfloat16 *q, *k_new, *v_new, *gate;
  const __nv_bfloat16 *q_norm_w, *k_norm_w;  // optional per-head RMSNorm weights [256] applied to q / k_new first
  __nv_bfloat16 *k_cache, *v_cache, *out;
  int64_t q_b, q_h, kn_b, kn_h, vn_b, vn_h, gate_b;
  int64_t kc_p, kc_h, kc_s, vc_p, vc_h, vc_s, bt_b;
  const int32_t* block_table;
  const int64_t* pos;
  const float* inv_freq;
  float* partials;
  int* counters;
  int* err;
  int batch, num_kv_heads, rotary_half, overlap;
  int partition;  // 0 = the time models below choose, 1 = stream-K, 2 = one whole segment per CTA, 3 = one segment
                  // per thread-block cluster
  int cluster_size;  // CTAs per cluster of this launch (1 = launched without clusters)
  float scale, eps;
};

// Position of a (sequence, kv head) segment on the unit line.  units = old pages + 1 (the appended token); [start, end)
// are its units.  Behind every segment the line has `gap` empty positions: a CTA stops at every segment boundary inside
// its range (merge of the eight warps, a partial or the output), which costs about as much as streaming `gap` units, so
// equal ranges of the line are ranges of equal TIME and a CTA with more boundaries gets fewer pages.
struct Segment {
  int b, h, start, end;
};

// cum[] is the exclusive prefix of (units + gap) per sequence.  A position inside a gap belongs to the segment before it
// (then u >= end).
__device__ __forceinline__ Segment segment_of_unit(int u, const int* cum, int batch, int heads, int gap) {
  int lo = 0, hi = batch - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (heads * cum[mid] <= u) lo = mid; else hi = mid - 1;
  }
  Segment s;
  s.b = lo;
  const int span = cum[lo + 1] - cum[lo];
  s.h = (u - heads * cum[lo]) / span;
  s.start = heads * cum[lo] + s.h * span;
  s.end = s.start + span - gap;
  return s;
}
__device__ __forceinline__ void segment_advance(Segment& s, const int* cum, int batch, int heads, int gap) {
  s.start = s.end + gap;
  if (++s.h == heads) {
    s.h = 0;
    ++s.b;
  }
  if (s.b < batch) s.end = s.start + (cum[s.b + 1] - cum[s.b]) - gap;
}

// One head row of q or k_new, 8 consecutive dims per lane (`w` = 4 packed bf16 pairs).
//
// Optional Qwen RMSNorm over the 256 dims, x * rsqrt(mean(x^2) + eps) * (1 + weight), rounded to bf16 as the
// reference's q_norm / k_norm output is a bf16 tensor (triton_kernels/qwen_rmsnorm.py:70-73, applied at
// engine/runner.py:476-489); the summation order is the one of add_rmsnorm_kernel, so both give the same bytes.
__device__ __forceinline__ void norm_row8(uint32_t (&w)[4], const __nv_bfloat16* weight, float eps, int lane) {
  const uint4 wraw = *reinterpret_cast<const uint4*>(weight + lane * 8);
  const uint32_t ww[4] = {wraw.x, wraw.y, wraw.z, wraw.w};
  float v[8];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = bf16_lo(w[i]);
    v[2 * i + 1] = bf16_hi(w[i]);
  }
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) ss = fmaf(v[j], v[j], ss);
  ss = warp_sum(ss);
  const float rs = rsqrtf(ss / static_cast<float>(HEAD_DIM) + eps);
#pragma unroll
  for (int i = 0; i < 4; ++i)
    w[i] = pack_bf16(v[2 * i] * rs * (1.0f + bf16_lo(ww[i])), v[2 * i + 1] * rs * (1.0f + bf16_hi(ww[i])));
}
// Partial RoPE of the row at position pos: dims [0, half) pair with [half, 2*half), angles = float(pos) * inv_freq[d] in
// fp32, full-range sincosf, result rounded to bf16 -- the arithmetic of triton_kernels/partial_rope.py:65-113.  Lanes
// [0, half/8) hold the first halves, the next half/8 lanes their partners; the other lanes pass through.
__device__ __forceinline__ void rope_row8(uint32_t (&w)[4], int half, const float* inv_freq, int64_t pos, int lane) {
  // half <= 32: one angle per lane; inv_freq may be a shared-memory copy
  if (half == 0) return;
  // the warp computes the `half` angles once, one sincosf per lane, and hands them round by shuffles
  float sn = 0.f, cs = 1.f;
  if (lane < half) sincosf(static_cast<float>(pos) * inv_freq[lane], &sn, &cs);
  const int lanes_half = half / 8;
  const bool in_rot = lane < 2 * lanes_half;
  const bool first = lane < lanes_half;
  const int partner = first ? lane + lanes_half : lane - lanes_half;
  const int dbase = (in_rot ? (first ? lane : partner) : 0) * 8;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t other = __shfl_sync(0xffffffffu, w[i], in_rot ? partner : lane);
    const float s0 = __shfl_sync(0xffffffffu, sn, dbase + 2 * i), c0 = __shfl_sync(0xffffffffu, cs, dbase + 2 * i);
    const float s1 = __shfl_sync(0xffffffffu, sn, dbase + 2 * i + 1), c1 = __shfl_sync(0xffffffffu, cs, dbase + 2 * i + 1);
    if (in_rot) {
      const uint32_t fa = first ? w[i] : other;  // first-half values
      const uint32_t fb = first ? other : w[i];  // second-half values
      float f0, g0, f1, g1;
      rope_pair(bf16_lo(fa), bf16_lo(fb), s0, c0, f0, g0);
      rope_pair(bf16_hi(fa), bf16_hi(fb), s1, c1, f1, g1);
      w[i] = first ? pack_bf16(f0, f1) : pack_bf16(g0, g1);
    }
  }
}

// Small read-only operands every CTA keeps in shared memory: a global load issued while the page copies saturate the
// memory system takes microseconds, and these are needed at every segment boundary.
struct FusedDecodeTables {
  float inv_freq[32];
  __align__(16) __nv_bfloat16 q_norm_w[HEAD_DIM];
  __align__(16) __nv_bfloat16 k_norm_w[HEAD_DIM];
  __align__(16) uint8_t new_rows[2 * HEAD_DIM * 2];  // k_new row | v_new row of the segment whose end is in this piece
};

// Stage the 4 Q heads of one segment in shared memory, normalised (optional) and rotated: warps 0-3 take one head
// each.  The caller synchronises.  The row is fetched by load_q_row() so that the caller can put the load in front of
// a burst of page copies (a small load issued behind them waits for the whole burst) and finish the row later.
__device__ __forceinline__ uint4 load_q_row(const FusedDecodeParams& p, int b, int h, int tid) {
  if (tid >= GROUP * 32) return make_uint4(0, 0, 0, 0);
  const int head = tid >> 5, lane = tid & 31;
  return *reinterpret_cast<const uint4*>(p.q + b * p.q_b + (h * GROUP + head) * p.q_h + lane * 8);
}
__device__ __forceinline__ void stage_q_row(__nv_bfloat16* buf, const FusedDecodeParams& p, const FusedDecodeTables& tb,
                                            const uint4& raw, int pos_b, int tid) {
  if (tid >= GROUP * 32) return;
  const int head = tid >> 5, lane = tid & 31;
  uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
  if (p.q_norm_w != nullptr) norm_row8(w, tb.q_norm_w, p.eps, lane);
  rope_row8(w, p.rotary_half, tb.inv_freq, pos_b, lane);
  *reinterpret_cast<uint4*>(buf + head * FD_Q_PITCH + lane * 8) = make_uint4(w[0], w[1], w[2], w[3]);
}
__device__ __forceinline__ void stage_q(__nv_bfloat16* buf, const FusedDecodeParams& p, const FusedDecodeTables& tb, int b,
                                        int h, int pos_b, int tid) {
  stage_q_row(buf, p, tb, load_q_row(p, b, h, tid), pos_b, tid);
}
__device__ __forceinline__ void cp_async16(void* dst_smem, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst_smem)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
// Asks the L2 for the q rows and the gate row of a segment ahead of their use (one 16-byte piece per thread of warps
// 0-3 and 8 bytes of gate per thread: the lines they touch cover both rows).
__device__ __forceinline__ void prefetch_l2(const void* ptr) {
  asm volatile("prefetch.global.L2 [%0];" ::"l"(ptr));
}

// The appended token as a one-row page: the normalised (optional), rotated k_new goes to row 0 of `k_tile` and to its
// slot in the cache (physical page `phys`).  Each lane owns 8 consecutive dims.  The raw rows were copied to
// tb.new_rows by this warp at the start of the piece (fetch_new_rows), so nothing here waits for global memory.
__device__ __forceinline__ void fetch_new_rows(FusedDecodeTables& tb, const FusedDecodeParams& p, int b, int h, int lane) {
  cp_async16(tb.new_rows + lane * 16, p.k_new + b * p.kn_b + h * p.kn_h + lane * 8);
  cp_async16(tb.new_rows + HEAD_DIM * 2 + lane * 16, p.v_new + b * p.vn_b + h * p.vn_h + lane * 8);
  cp_async_commit();
}
__device__ __forceinline__ void stage_new_k(uint8_t* k_tile, const FusedDecodeParams& p, const FusedDecodeTables& tb, int h,
                                            int64_t pos_b, int64_t phys, int lane) {
  cp_async_wait_all();
  __syncwarp();
  const uint4 kraw = *reinterpret_cast<const uint4*>(tb.new_rows + lane * 16);
  uint32_t kw[4] = {kraw.x, kraw.y, kraw.z, kraw.w};
  if (p.k_norm_w != nullptr) norm_row8(kw, tb.k_norm_w, p.eps, lane);
  rope_row8(kw, p.rotary_half, tb.inv_freq, pos_b, lane);
  const uint4 krot = make_uint4(kw[0], kw[1], kw[2], kw[3]);
  *reinterpret_cast<uint4*>(k_tile + tile_offset<true>(0, lane)) = krot;
  *reinterpret_cast<uint4*>(p.k_cache + phys * p.kc_p + h * p.kc_h + (pos_b % PAGE) * p.kc_s + lane * 8) = krot;
}
__device__ __forceinline__ void stage_new_v(uint8_t* v_tile, const FusedDecodeParams& p, const FusedDecodeTables& tb, int h,
                                            int64_t pos_b, int64_t phys, int lane) {
  const uint4 vraw = *reinterpret_cast<const uint4*>(tb.new_rows + HEAD_DIM * 2 + lane * 16);
  *reinterpret_cast<uint4*>(v_tile + tile_offset<true>(0, lane)) = vraw;
  *reinterpret_cast<uint4*>(p.v_cache + phys * p.vc_p + h * p.vc_h + (pos_b % PAGE) * p.vc_s + lane * 8) = vraw;
}

// out = bf16( bf16(acc / l) * sigmoid(gate) ), 4 consecutive dims of one head per thread; without a gate (p.gate NULL)
// out = bf16(acc / l), the output of the reference's combine kernel.
__device__ __forceinline__ void finish_store(const FusedDecodeParams& p, int b, int hq, int d0, const float (&acc)[4],
                                             float l, uint2 gv) {
  const int64_t col = static_cast<int64_t>(hq) * HEAD_DIM + d0;
  if (p.gate == nullptr) {
    const int64_t row = static_cast<int64_t>(p.num_kv_heads) * GROUP * HEAD_DIM;
    *reinterpret_cast<uint2*>(p.out + b * row + col) = make_uint2(pack_bf16(acc[0] / l, acc[1] / l), pack_bf16(acc[2] / l, acc[3] / l));
    return;
  }
  const float inv_l = 1.f / l;
  const float x0 = round_bf16(acc[0] * inv_l), x1 = round_bf16(acc[1] * inv_l);
  const float x2 = round_bf16(acc[2] * inv_l), x3 = round_bf16(acc[3] * inv_l);
  const float g0 = 1.f / (1.f + __expf(-bf16_lo(gv.x))), g1 = 1.f / (1.f + __expf(-bf16_hi(gv.x)));
  const float g2 = 1.f / (1.f + __expf(-bf16_lo(gv.y))), g3 = 1.f / (1.f + __expf(-bf16_hi(gv.y)));
  const int64_t row = static_cast<int64_t>(p.num_kv_heads) * GROUP * HEAD_DIM;
  *reinterpret_cast<uint2*>(p.out + b * row + col) = make_uint2(pack_bf16(x0 * g0, x1 * g1), pack_bf16(x2 * g2, x3 * g3));
}

// Fold one exported state (m, l, acc) into a running one with the usual max-rescaling.
__device__ __forceinline__ void merge_state(float& m_run, float& l_run, float (&acc)[4], float m_in, float l_in,
                                            const float4& x) {
  if (m_in == -INFINITY) return;  // empty contribution
  const float m_new = fmaxf(m_run, m_in);
  const float s_old = (m_run == -INFINITY) ? 0.f : __expf(m_run - m_new);
  const float s_in = __expf(m_in - m_new);
  l_run = l_run * s_old + l_in * s_in;
  acc[0] = acc[0] * s_old + x.x * s_in;
  acc[1] = acc[1] * s_old + x.y * s_in;
  acc[2] = acc[2] * s_old + x.z * s_in;
  acc[3] = acc[3] * s_old + x.w * s_in;
  m_run = m_new;
}

__global__ void __launch_bounds__(FD_THREADS, 1)
fused_decode_kernel(const __grid_constant__ FusedDecodeParams p, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_v) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ uint64_t bars[FD_WARPS][FD_RING];
  __shared__ int s_last;
  __shared__ int s_max_units;
  __shared__ FusedDecodeTables tb;
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* merge = reinterpret_cast<float*>(smem + FD_SMEM_RING);
  int* cum = reinterpret_cast<int*>(smem + FD_SMEM_RING + FD_SMEM_MERGE);
  int* pos_s = reinterpret_cast<int*>(smem + FD_SMEM_RING + FD_SMEM_MERGE + FD_SMEM_CUM);
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smem + FD_SMEM_RING + FD_SMEM_MERGE + FD_SMEM_CUM + FD_SMEM_POS);
  float* recv = reinterpret_cast<float*>(smem + FD_SMEM_RING + FD_SMEM_MERGE + FD_SMEM_CUM + FD_SMEM_POS + FD_SMEM_Q);
  float* recv_ml = recv + FD_TILE_FLOATS;   // [source rank][m[4], l[4]]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int heads = p.num_kv_heads, batch = p.batch, gap = p.gap;
  uint8_t* ring = smem + warp * FD_RING * TILE_BYTES_SW;
  if (lane == 0) {
    for (int s = 0; s < FD_RING; ++s) mbar_init(&bars[warp][s], 1);
    mbar_fence_init();
  }
  if (tid == 0) {
    prefetch_tensormap(&map_k);
    prefetch_tensormap(&map_v);
  }
  if (p.overlap & OVERLAP_TRIGGER) pdl_trigger();  // the successor may start: it waits for this grid before it reads `out`
  // Started early (programmatic dependent launch): with the PREFETCH flag the position prefix, the page-id gathers and
  // the first K/V page copies below overlap with the predecessor (it must not write pos, the block table or the
  // caches); q, k_new, v_new and gate are the predecessor's output and are read only after the wait further down.
  if (!(p.overlap & OVERLAP_PREFETCH)) pdl_wait();

  // weights and frequencies are nobody's output: staged before anything else, published by the barrier below
  if (warp == 7) tb.inv_freq[lane] = lane < p.rotary_half ? p.inv_freq[lane] : 0.f;
  if (warp == 6 && p.q_norm_w != nullptr)
    *reinterpret_cast<uint4*>(tb.q_norm_w + lane * 8) = *reinterpret_cast<const uint4*>(p.q_norm_w + lane * 8);
  if (warp == 5 && p.k_norm_w != nullptr)
    *reinterpret_cast<uint4*>(tb.k_norm_w + lane * 8) = *reinterpret_cast<const uint4*>(p.k_norm_w + lane * 8);
  // ---- exclusive prefix of units per sequence: units_b = cdiv(pos[b], 16) + 1
  for (int b = tid; b < batch; b += FD_THREADS) {
    const int pb = static_cast<int>(p.pos[b]);
    pos_s[b] = pb;
    cum[b + 1] = (pb + PAGE - 1) / PAGE + 1 + gap;
  }
  __syncthreads();
  if (warp == 0) {
    int carry = 0, longest = 0;
    for (int base = 0; base < batch; base += 32) {
      const int idx = base + lane;
      int v = (idx < batch) ? cum[idx + 1] : 0;
      longest = max(longest, v);
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += n;
      }
      if (idx < batch) cum[idx + 1] = v + carry;
      carry += __shfl_sync(0xffffffffu, v, 31);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) longest = max(longest, __shfl_xor_sync(0xffffffffu, longest, o));
    if (lane == 0) {
      cum[0] = 0;
      s_max_units = longest - gap;
    }
  }
  __syncthreads();

  // Three ways to cut the work.
  //  - Stream-K: equal ranges of the unit line per CTA (never less than one position per warp: tiny problems use fewer
  //    CTAs and leave fewer partials to merge).  A segment cut by a range boundary costs a partial, a ticket and a
  //    merge, and a CTA that spans several segments stops at every boundary; the gap behind every segment on the line
  //    charges a range for the boundaries inside it, so that the ranges take equal time rather than hold equal pages.
  //  - One whole segment per CTA, when there are no more segments than CTAs: no partials at all, but the longest
  //    segment sets the time, and an SM alone streams at about 75 GB/s.
  //  - One segment per CLUSTER (launches with clusters only, when every segment gets a cluster of its own): the CTAs
  //    of a cluster take equal shares of the segment's units and merge through distributed shared memory.
  // The choice compares time models fitted to measurements of this kernel on B200 (nanoseconds, u = units of 16 KiB;
  // every form is also bound by the DRAM rate, 2.64 ns per unit):
  //    stream-K  max(300 line positions per CTA, 2.64 u_total) + 8000 + 180 u_longest / (positions per CTA)
  //              (the last term: partials the longest segment leaves for its final merge)
  //    whole     max(165 u_longest, 2.64 u_total) + 8500
  //    cluster   max(190 u_longest / cluster_size, 2.64 u_total) + 8500
  // A form is taken over stream-K when its model wins by 5 %.
  const int total = heads * cum[batch];  // length of the line, gaps included
  const int grid = static_cast<int>(gridDim.x), nseg = batch * heads;
  const int chunk = max((total + grid - 1) / grid, FD_WARPS);
  const int csize = p.cluster_size;
  const int dram = (total - nseg * gap) * 66 / 25;  // 2.64 ns per unit
  const int t_stream = max(300 * chunk, dram) + 8000 + 180 * s_max_units / chunk;
  const int t_whole = max(165 * s_max_units, dram) + 8500;
  const int t_cluster = max(190 * ((s_max_units + csize - 1) / csize), dram) + 8500;
  const bool cluster_fits = csize > 1 && nseg * csize <= grid;
  const bool whole_fits = nseg <= grid;
  int form = 1;  // 1 stream-K, 2 whole segments, 3 cluster per segment
  if (p.partition != 0) {
    form = (p.partition == 3 && cluster_fits) ? 3 : (p.partition == 2 && whole_fits) ? 2 : 1;
  } else {
    int best = t_stream;
    if (whole_fits && 21 * t_whole < 20 * best) {
      form = 2;
      best = t_whole;
    }
    if (cluster_fits && 21 * t_cluster < 20 * t_stream && t_cluster <= best) form = 3;
  }
  const bool cluster_mode = form == 3, whole_segments = form == 2;
  int r0, r1;
  Segment cseg = {0, 0, 0, 0};  // cluster mode: the segment of this CTA's cluster
  const int rank = csize > 1 ? static_cast<int>(blockIdx.x) % csize : 0;  // == %cluster_ctarank of a 1-D cluster
  if (cluster_mode) {
    const int cl = static_cast<int>(blockIdx.x) / csize;
    if (cl < nseg) {
      const int sb = cl / heads, sh = cl % heads;
      const int span = cum[sb + 1] - cum[sb], units = span - gap;
      const int per = (units + csize - 1) / csize;
      const int start = heads * cum[sb] + sh * span;
      cseg.b = sb;
      cseg.h = sh;
      cseg.start = start;
      cseg.end = start + units;
      r0 = min(start + rank * per, start + units);
      r1 = min(r0 + per, start + units);
    } else {
      pdl_wait();  // a cluster without a segment: all its CTAs leave together, nobody waits for them
      return;
    }
  } else if (whole_segments) {
    if (static_cast<int>(blockIdx.x) < nseg) {
      const int sb = blockIdx.x / heads, sh = blockIdx.x % heads;
      const int span = cum[sb + 1] - cum[sb];
      r0 = heads * cum[sb] + sh * span;
      r1 = r0 + span - gap;
    } else {
      r0 = r1 = total;
    }
  } else {
    r0 = blockIdx.x * chunk;
    r1 = min(r0 + chunk, total);
  }
  if (r0 >= r1 && !cluster_mode) {
    pdl_wait();  // an idle CTA still orders the grid after its predecessor
    return;
  }
  // (in cluster mode a CTA without units of its own still takes part in the exchange below: the cluster barrier needs
  //  every thread of every CTA of the cluster, and this CTA finishes a slice of the output)
  Segment seg0 = cluster_mode ? cseg : segment_of_unit(r0, cum, batch, heads, gap);
  if (!cluster_mode) {
    if (r0 >= seg0.end) segment_advance(seg0, cum, batch, heads, gap);  // the range starts inside a gap
    if (seg0.start >= r1) {                                             // ... and ends in it
      pdl_wait();
      return;
    }
  }

  // ---- per-warp issue cursor: walks the same unit sequence as the consumer, FD_RING tiles ahead.
  // Tile sequence of a warp: K(u0), V(u0), K(u1), V(u1), ...; tile n lives in ring slot n % FD_RING.
  Segment iseg = seg0;
  int iu = max(r0, seg0.start) + warp;  // unit whose tiles are issued next
  bool i_is_v = false;       // next tile to issue is the V tile of unit iu
  int ii = 0;                // index of unit iu among this warp's units of the current piece
  int win_base = -1;         // first ii covered by the page-id window (-1 = none loaded)
  int win_phys = 0;          // lane L holds the physical page of this warp's (win_base + L)-th unit of the piece
  int pre_phys = 0;          // the window this warp needs next, asked for when the current one was loaded: a gather
  int pre_key = -1;          // issued while the page copies saturate memory takes microseconds (key = its first unit)
  int cur_phys = 0;
  int issued = 0, consumed = 0;
  uint32_t phase_bits = 0;
  bool dead = false;

  auto issue_next = [&]() {
    for (;;) {
      const int hi = min(iseg.end, r1);
      if (iu < hi) {
        const int j = iu - iseg.start;
        const int np = iseg.end - iseg.start - 1;
        const int slot = issued % FD_RING;
        if (j < np) {
          if (!i_is_v) {
            if (win_base < 0 || ii - win_base >= 32) {
              // one gather of the next 32 page ids of this warp (stride FD_WARPS in the table row) ...
              win_base = ii;
              if (pre_key == iu) {
                win_phys = pre_phys;
              } else {
                const int jl = j + lane * FD_WARPS;
                win_phys = (iu + lane * FD_WARPS < hi && jl < np) ? p.block_table[iseg.b * p.bt_b + jl] : 0;
              }
              // ... and, not waited for, the one after it: the same segment 32 units of this warp further on, or the
              // warp's first units of the next segment in the range
              Segment ns = iseg;
              int nu = iu + 32 * FD_WARPS;
              if (nu >= hi && iseg.end + gap < r1) {
                segment_advance(ns, cum, batch, heads, gap);
                nu = ns.start + warp;
              }
              const int nhi = min(ns.end, r1), njl = nu - ns.start + lane * FD_WARPS;
              pre_key = nu < nhi ? nu : -1;
              if (pre_key >= 0)
                pre_phys = (nu + lane * FD_WARPS < nhi && njl < ns.end - ns.start - 1) ? p.block_table[ns.b * p.bt_b + njl] : 0;
            }
            cur_phys = __shfl_sync(0xffffffffu, win_phys, ii - win_base);
          }
          // the cache as a matrix of token rows: row = (page * H_kv + head) * 16 + slot; one box = one page of one head
          if (lane == 0) {
            const int row0 = (cur_phys * heads + iseg.h) * PAGE;
            mbar_expect_tx(&bars[warp][slot], TILE_TX_BYTES);
            tma_load_3d(ring + slot * TILE_BYTES_SW, i_is_v ? &map_v : &map_k, 0, row0, 0, &bars[warp][slot]);
          }
        }
        ++issued;
        if (i_is_v) {
          iu += FD_WARPS;
          ++ii;
        }
        i_is_v = !i_is_v;
        return;
      }
      if (iseg.end + gap >= r1) return;  // no further segment starts inside this CTA's range
      segment_advance(iseg, cum, batch, heads, gap);
      iu = iseg.start + warp;
      ii = 0;
      win_base = -1;
    }
  };
  __syncwarp();
  // The first segment's q rows: fetched BEFORE the burst of page copies when the predecessor has already finished
  // (behind 148 x 24 copies the load would wait for all of them); with the PREFETCH flag q is not final yet and is read
  // after the wait below.
  const bool q_early = !(p.overlap & OVERLAP_PREFETCH);
  uint4 q_raw = make_uint4(0, 0, 0, 0);
  if (q_early) q_raw = load_q_row(p, seg0.b, seg0.h, tid);
  if (seg0.end + gap < r1 && tid < GROUP * 32) {  // the second piece's q rows: into the L2 ahead of their staging
    Segment nxt = seg0;
    segment_advance(nxt, cum, batch, heads, gap);
    prefetch_l2(p.q + nxt.b * p.q_b + (nxt.h * GROUP + warp) * p.q_h + lane * 8);
  }
  for (int s = 0; s < FD_RING; ++s) issue_next();

  // ---- consumer: CTA-uniform loop over the pieces of this range
  Segment seg = seg0;
  const int hh = tid >> 6, d0 = (tid & 63) * 4;  // element mapping of the merge / finish steps
  int piece = 0;
  bool have_pending = false;
  Segment pend_seg = seg;
  int pend_first = 0, pend_last = 0;
  uint2 pend_gate = make_uint2(0, 0);
  // merge the partials CTAs [c_first, c_last] left for segment `sg` and finish it
  auto combine_and_finish = [&](const Segment& sg, int c_first, int c_last, uint2 gate_bits) {
    __threadfence();
    float m_fin = -INFINITY, l_fin = 0.f;
    float a4[4] = {0.f, 0.f, 0.f, 0.f};
    // eight contributors per round: all their loads are in flight before the first dependent merge
    for (int c0 = c_first; c0 <= c_last; c0 += 8) {
      float mm[8], ll[8];
      float4 xx[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int c = min(c0 + i, c_last);
        const float* src = p.partials + (static_cast<int64_t>(c) * 2 + (c == c_first ? 1 : 0)) * FD_PARTIAL_FLOATS;
        mm[i] = __ldcg(src + hh);
        ll[i] = __ldcg(src + 4 + hh);
        xx[i] = __ldcg(reinterpret_cast<const float4*>(src + 8 + hh * HEAD_DIM + d0));
      }
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (c0 + i <= c_last) merge_state(m_fin, l_fin, a4, mm[i], ll[i], xx[i]);
    }
    finish_store(p, sg.b, sg.h * GROUP + hh, d0, a4, l_fin, gate_bits);
  };
  pdl_wait();  // from here on the predecessor's q / k_new / v_new / gate are read and global memory is written
  if (!q_early) q_raw = load_q_row(p, seg.b, seg.h, tid);
  stage_q_row(q_s, p, tb, q_raw, pos_s[seg.b], tid);
  __syncthreads();
  while (seg.start < r1 || (cluster_mode && piece == 0)) {  // in cluster mode exactly once, also without units
    const int lo = max(seg.start, r0), hi = min(seg.end, r1);
    const int np = seg.end - seg.start - 1;
    const int64_t pos_b = pos_s[seg.b];
    // the gate row of this segment is only needed at the very end: fetch it now, off the critical path
    const uint2 gate_pf = p.gate == nullptr ? make_uint2(0, 0)
                                            : *reinterpret_cast<const uint2*>(p.gate + seg.b * p.gate_b +
                                                                              static_cast<int64_t>(seg.h * GROUP + hh) * HEAD_DIM + d0);
    // rotated Q of the NEXT piece goes to the other buffer while this piece streams (published by the merge barriers)
    // (its rows were asked into the L2 one piece earlier: a load that misses there queues behind the page copies)
    if (seg.end + gap < r1) {  // another segment starts inside the range
      Segment nxt = seg;
      segment_advance(nxt, cum, batch, heads, gap);
      if (nxt.end + gap < r1 && tid < GROUP * 32) {
        Segment nn = nxt;
        segment_advance(nn, cum, batch, heads, gap);
        prefetch_l2(p.q + nn.b * p.q_b + (nn.h * GROUP + warp) * p.q_h + lane * 8);
      }
      stage_q(q_s + ((piece + 1) & 1) * GROUP * FD_Q_PITCH, p, tb, nxt.b, nxt.h, pos_s[nxt.b], tid);
    }
    // the appended token's rows and its page: asked for now by the warp that will reach the segment's last unit
    int64_t new_phys = 0;
    if (hi == seg.end && hi > lo && warp == (seg.end - 1 - lo) % FD_WARPS) {
      fetch_new_rows(tb, p, seg.b, seg.h, lane);
      new_phys = p.block_table[seg.b * p.bt_b + pos_b / PAGE];
    }
    DecodeWarpState st;
    decode_state_init(st);
    if (lo + warp < hi) decode_load_q(st, q_s + (piece & 1) * GROUP * FD_Q_PITCH, FD_Q_PITCH, lane);
    for (int u = lo + warp; u < hi; u += FD_WARPS) {
      const int j = u - seg.start;
      const bool is_page = j < np;
      const int valid = is_page ? min(PAGE, static_cast<int>(pos_b) - j * PAGE) : 1;
      uint32_t b0 = 0, b1 = 0;
      float alpha0 = 1.f, alpha1 = 1.f;
#pragma unroll
      for (int part = 0; part < 2; ++part) {
        const int slot = consumed % FD_RING;
        uint8_t* tile = ring + slot * TILE_BYTES_SW;
        bool ready = !dead;
        if (is_page) {
          if (ready) {
            if (mbar_wait_bounded(&bars[warp][slot], (phase_bits >> slot) & 1u)) {
              phase_bits ^= (1u << slot);
            } else {
              dead = true;
              ready = false;
              if (lane == 0) atomicExch(p.err, 1);
            }
          }
        } else {
          if (part == 0) stage_new_k(tile, p, tb, seg.h, pos_b, new_phys, lane);
          else stage_new_v(tile, p, tb, seg.h, pos_b, new_phys, lane);
          __syncwarp();
        }
        if (ready) {
          if (part == 0) decode_scores<true>(st, tile, valid, p.scale, lane, b0, b1, alpha0, alpha1);
          else decode_accumulate<true>(st, tile, valid, b0, b1, alpha0, alpha1, lane);
        }
        ++consumed;
        // generic-proxy writes to this slot (row clears of a partly filled page, the appended token) are ordered before
        // the next bulk copy into it; a full page was only read
        if (valid < PAGE) fence_proxy_async();
        __syncwarp();
        if (!dead) issue_next();
      }
    }
    decode_reduce_l(st);

    // ---- merge the eight warps' states, four at a time
    float m_all = -INFINITY, l_all = 0.f;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int round = 0; round < FD_WARPS / FD_MERGE_SLOTS; ++round) {
      if ((warp / FD_MERGE_SLOTS) == round) {
        float* mine = merge + (warp % FD_MERGE_SLOTS) * FD_PARTIAL_FLOATS;
        if (lane < 2) {
          mine[lane * 2] = st.m[0];
          mine[lane * 2 + 1] = st.m[1];
          mine[4 + lane * 2] = st.l[0];
          mine[4 + lane * 2 + 1] = st.l[1];
        }
        decode_store_acc_smem(st, mine + 8, lane);
      }
      __syncthreads();
#pragma unroll
      for (int w = 0; w < FD_MERGE_SLOTS; ++w) {
        const float* src = merge + w * FD_PARTIAL_FLOATS;
        merge_state(m_all, l_all, acc, src[hh], src[4 + hh],
                    *reinterpret_cast<const float4*>(src + 8 + hh * HEAD_DIM + d0));
      }
      __syncthreads();  // merge buffer free again
    }

    // a partial left by the previous piece: its arrival ticket was taken by thread 0 while this piece streamed
    if (have_pending) {
      if (s_last) combine_and_finish(pend_seg, pend_first, pend_last, pend_gate);
      have_pending = false;
    }
    const bool whole = (lo == seg.start) && (hi == seg.end);
    if (cluster_mode) {
      // ---- exchange through distributed shared memory.  Output element e = tid (4 dims of one head) is finished by
      // the CTA of rank e / tpr; every CTA sends each of its 1024 accumulators to the rank that finishes it (slot
      // [own rank][e % tpr] of that CTA's receive buffer) and its (m, l) to everybody, then all meet at the barrier.
      const int tpr = FD_THREADS / csize;
      const uint32_t slot = smem_u32(recv + (rank * tpr + (tid % tpr)) * 4);
      st_cluster_f32x4(cluster_map(slot, static_cast<uint32_t>(tid / tpr)), acc[0], acc[1], acc[2], acc[3]);
      if ((tid & 63) == 0) {
        for (int dst = 0; dst < csize; ++dst) {
          const uint32_t ml = cluster_map(smem_u32(recv_ml + rank * 8), static_cast<uint32_t>(dst));
          asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(ml + hh * 4), "f"(m_all) : "memory");
          asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(ml + 16 + hh * 4), "f"(l_all) : "memory");
        }
      }
      cluster_sync();  // release / acquire: every CTA's slices and (m, l) have landed
      if (tid / tpr == rank) {
        float m_fin = -INFINITY, l_fin = 0.f;
        float a4[4] = {0.f, 0.f, 0.f, 0.f};
        for (int src = 0; src < csize; ++src)
          merge_state(m_fin, l_fin, a4, recv_ml[src * 8 + hh], recv_ml[src * 8 + 4 + hh],
                      *reinterpret_cast<const float4*>(recv + (src * tpr + (tid % tpr)) * 4));
        finish_store(p, seg.b, seg.h * GROUP + hh, d0, a4, l_fin, gate_pf);
      }
    } else if (whole) {
      finish_store(p, seg.b, seg.h * GROUP + hh, d0, acc, l_all, gate_pf);
    } else {
      // ---- leave a partial; the last CTA to arrive on this segment merges all of them.  Nobody waits for the
      // ticket here: the result is looked at after the next piece's merge barriers (or after the loop).
      const int which = (seg.start < r0) ? 0 : 1;
      float* dst = p.partials + (static_cast<int64_t>(blockIdx.x) * 2 + which) * FD_PARTIAL_FLOATS;
      if ((tid & 63) == 0) {
        dst[hh] = m_all;
        dst[4 + hh] = l_all;
      }
      *reinterpret_cast<float4*>(dst + 8 + hh * HEAD_DIM + d0) = make_float4(acc[0], acc[1], acc[2], acc[3]);
      pend_seg = seg;
      pend_first = seg.start / chunk;
      pend_last = (seg.end - 1) / chunk;
      pend_gate = gate_pf;
      have_pending = true;
      __syncthreads();  // every thread's partial stores happen-before thread 0's release below
      if (tid == 0) {
        __threadfence();
        const int seg_id = seg.b * heads + seg.h;
        const int old = atomicAdd(p.counters + seg_id, 1);
        const int last = (old == pend_last - pend_first);
        if (last) p.counters[seg_id] = 0;  // ready for the next launch
        s_last = last;
      }
    }
    segment_advance(seg, cum, batch, heads, gap);
    ++piece;
  }
  if (have_pending) {
    __syncthreads();
    if (s_last) combine_and_finish(pend_seg, pend_first, pend_last, pend_gate);
  }
  if (dead) {
    for (int s = 0; s < FD_RING; ++s) mbar_wait_bounded(&bars[warp][s], (phase_bits >> s) & 1u, 1u << 12);
  }
}

}  // namespace b200

using namespace b200;

// Tensor maps of the KV pools seen as matrices of token rows [rows][256]; a box is one page of one head
// ({64 dims, 16 rows, 4 column blocks}).  Encoding costs a few microseconds of host time, so the last few
// (pointer, rows) pairs are remembered: a model has a fixed set of pools.  The table is shared by all host threads:
// it is searched and filled under a mutex and the map is copied out, so a concurrent caller cannot overwrite an entry
// between the look-up and the launch.
static bool cache_tile_map(const void* base, int64_t rows, CUtensorMap* out) {
  static std::mutex mu;
  std::lock_guard<std::mutex> lock(mu);
  struct Entry {
    const void* base;
    int64_t rows;
    int dev;
    CUtensorMap map;
  };
  constexpr int N = 32;
  static Entry entries[N];
  static int used = 0, next = 0;
  int dev = 0;
  cudaGetDevice(&dev);
  for (int i = 0; i < used; ++i)
    if (entries[i].base == base && entries[i].rows == rows && entries[i].dev == dev) {
      *out = entries[i].map;
      return true;
    }
  Entry& e = entries[next];
  e.base = nullptr;  // not a valid entry while it is being rewritten
  if (!encode_tile_map(&e.map, base, static_cast<uint64_t>(rows), HEAD_DIM, HEAD_DIM * 2, PAGE, HEAD_DIM / 64)) return false;
  e.base = base;
  e.rows = rows;
  e.dev = dev;
  next = (next + 1) % N;
  if (used < N) ++used;
  *out = e.map;
  return true;
}

extern "C" int64_t b200_fused_decode_workspace_bytes(void) { return FD_WORKSPACE_BYTES; }

// CTAs of the fused kernel that can be resident at once when launched in clusters of `csize` (asked from the runtime
// once per device and size; 0 when such clusters cannot be launched).  Sizes above 8 need the kernel's opt-in.
static int cluster_limit(int csize) {
  static int cached[64][5];       // [device][log2(csize)]: 0 = unknown, -1 = cannot launch
  static std::mutex mu;
  int dev = 0, lg = 0;
  while ((1 << lg) < csize) ++lg;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64 || lg > 4) return 0;
  std::lock_guard<std::mutex> lock(mu);
  if (cached[dev][lg] == 0) {
    cached[dev][lg] = -1;
    bool ok = true;
    if (csize > 8)
      ok = cudaFuncSetAttribute(fused_decode_kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess;
    if (ok) {
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(static_cast<unsigned>(csize) * 16);
      cfg.blockDim = dim3(FD_THREADS);
      cfg.dynamicSmemBytes = FD_SMEM_TOTAL;
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = static_cast<unsigned>(csize);
      attr[0].val.clusterDim.y = 1;
      attr[0].val.clusterDim.z = 1;
      cfg.attrs = attr;
      cfg.numAttrs = 1;
      int clusters = 0;
      if (cudaOccupancyMaxActiveClusters(&clusters, fused_decode_kernel, &cfg) == cudaSuccess && clusters > 0)
        cached[dev][lg] = clusters * csize;
    }
    cudaGetLastError();  // a refused query must not look like a failed launch later
  }
  return cached[dev][lg] > 0 ? cached[dev][lg] : 0;
}

static int fused_decode_impl(const void* q, int64_t q_stride_b, int64_t q_stride_h, const void* k_new,
                                           int64_t kn_stride_b, int64_t kn_stride_h, const void* v_new,
                                           int64_t vn_stride_b, int64_t vn_stride_h, const void* gate,
                                           int64_t gate_stride_b, void* k_cache, void* v_cache, int64_t kc_stride_p,
                                           int64_t kc_stride_h, int64_t kc_stride_s, int64_t vc_stride_p,
                                           int64_t vc_stride_h, int64_t vc_stride_s, int64_t num_pages,
                                           const int32_t* block_table, int64_t bt_stride_b, const int64_t* pos,
                                           const float* inv_freq, int32_t rotary_dim, void* out, void* workspace,
                                           int32_t batch, int32_t num_q_heads, int32_t num_kv_heads, int32_t head_dim,
                                           const void* q_norm_weight, const void* k_norm_weight, float eps,
                                           int32_t overlap, int32_t partition, b200_stream_t stream) {
  B200_REQUIRE(partition >= 0 && partition <= 3, "fused_decode_attention: partition must be 0..3 (got %d)", partition);
  B200_REQUIRE(aligned16(q_norm_weight) && aligned16(k_norm_weight),
               "fused_decode_attention: norm weights must be 16-byte aligned");
  B200_REQUIRE(batch > 0 && batch <= FD_MAX_BATCH, "fused_decode_attention: batch must be in [1, %d] (got %d)",
               FD_MAX_BATCH, batch);
  B200_REQUIRE(head_dim == HEAD_DIM, "fused_decode_attention: head_dim must be %d (got %d)", HEAD_DIM, head_dim);
  B200_REQUIRE(num_kv_heads > 0 && num_q_heads == num_kv_heads * GROUP && batch * num_kv_heads <= FD_MAX_SEGMENTS,
               "fused_decode_attention: needs %d Q heads per KV head and batch*H_kv <= %d", GROUP, FD_MAX_SEGMENTS);
  B200_REQUIRE(rotary_dim == 0 || rotary_dim == 64, "fused_decode_attention: rotary_dim must be 64 or 0 (got %d)",
               rotary_dim);
  B200_REQUIRE(rotary_dim == 0 || inv_freq != nullptr, "fused_decode_attention: inv_freq is NULL");
  B200_REQUIRE(workspace != nullptr && (reinterpret_cast<uintptr_t>(workspace) % 256 == 0),
               "fused_decode_attention: workspace must be 256-byte aligned");
  const bool strides_ok = (q_stride_b % 8 == 0) && (q_stride_h % 8 == 0) && (kn_stride_b % 8 == 0) &&
                          (kn_stride_h % 8 == 0) && (vn_stride_b % 8 == 0) && (vn_stride_h % 8 == 0) &&
                          (gate_stride_b % 8 == 0) && (kc_stride_p % 8 == 0) && (kc_stride_h % 8 == 0) &&
                          (kc_stride_s % 8 == 0) && (vc_stride_p % 8 == 0) && (vc_stride_h % 8 == 0) &&
                          (vc_stride_s % 8 == 0);
  B200_REQUIRE(strides_ok && aligned16(q) && aligned16(k_new) && aligned16(v_new) && aligned16(gate) &&
                   aligned16(k_cache) && aligned16(v_cache) && aligned16(out),
               "fused_decode_attention: tensors must be 16-byte aligned with strides that are multiples of 8");
  // the pages are fetched with tensor-map TMA: the pools must be the dense [num_pages, H_kv, 16, 256] layout that
  // the reference allocates (triton_kernels/gqa_attention_decode_paged.py:100-111)
  const int64_t dense_h = static_cast<int64_t>(PAGE) * HEAD_DIM, dense_p = dense_h * num_kv_heads;
  B200_REQUIRE(num_pages > 0 && kc_stride_s == HEAD_DIM && vc_stride_s == HEAD_DIM && kc_stride_h == dense_h &&
                   vc_stride_h == dense_h && kc_stride_p == dense_p && vc_stride_p == dense_p,
               "fused_decode_attention: k_cache / v_cache must be contiguous [num_pages, H_kv, 16, 256]");
  CUtensorMap map_k, map_v;
  if (!cache_tile_map(k_cache, num_pages * num_kv_heads * PAGE, &map_k) ||
      !cache_tile_map(v_cache, num_pages * num_kv_heads * PAGE, &map_v))
    return fail(ERR_RUNTIME, "fused_decode_attention: cannot encode the cache tensor maps");
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    if (cudaFuncSetAttribute(fused_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FD_SMEM_TOTAL) !=
        cudaSuccess)
      return fail(ERR_RUNTIME, "fused_decode_attention: cannot raise dynamic shared memory to %d", FD_SMEM_TOTAL);
    configured[dev] = true;
  }
  FusedDecodeParams p;
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.k_new = static_cast<const __nv_bfloat16*>(k_new);
  p.v_new = static_cast<const __nv_bfloat16*>(v_new);
  p.gate = static_cast<const __nv_bfloat16*>(gate);
  p.k_cache = static_cast<__nv_bfloat16*>(k_cache);
  p.v_cache = static_cast<__nv_bfloat16*>(v_cache);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.q_b = q_stride_b; p.q_h = q_stride_h;
  p.kn_b = kn_stride_b; p.kn_h = kn_stride_h;
  p.vn_b = vn_stride_b; p.vn_h = vn_stride_h;
  p.gate_b = gate_stride_b;
  p.kc_p = kc_stride_p; p.kc_h = kc_stride_h; p.kc_s = kc_stride_s;
  p.vc_p = vc_stride_p; p.vc_h = vc_stride_h; p.vc_s = vc_stride_s;
  p.bt_b = bt_stride_b;
  p.block_table = block_table;
  p.pos = pos;
  p.inv_freq = inv_freq;
  p.counters = static_cast<int*>(workspace);
  p.partials = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + FD_COUNTER_BYTES);
  p.err = wait_timeout_flag();
  if (!p.err) return fail(ERR_RUNTIME, "fused_decode_attention: no error flag");
  p.batch = batch;
  p.num_kv_heads = num_kv_heads;
  p.rotary_half = rotary_dim / 2;
  p.overlap = overlap;
  p.q_norm_w = static_cast<const __nv_bfloat16*>(q_norm_weight);
  p.k_norm_w = static_cast<const __nv_bfloat16*>(k_norm_weight);
  p.eps = eps;
  p.scale = 1.0f / sqrtf(static_cast<float>(head_dim));
  int grid = sm_count();
  if (grid > FD_MAX_CTAS) grid = FD_MAX_CTAS;
  // Up to 64 segments: launch as clusters so that the kernel may give every segment a whole cluster (the largest power
  // of two that still leaves each segment its own cluster, at most 16).  The cluster size depends on the batch only,
  // so it is the same for every replay of a captured launch; whether the cluster form is used is decided on the
  // device from the lengths.  cluster_limit(): how many CTAs of a cluster size can be resident at once.
  const int nseg = batch * num_kv_heads;
  int csize = 1;
  if (nseg <= 64) {
    csize = FD_MAX_CLUSTER;
    while (csize > 1 && (nseg * csize > grid || cluster_limit(csize) < nseg * csize)) csize >>= 1;
  }
  B200_REQUIRE(partition != 2 || nseg <= grid,
               "fused_decode_attention: partition 2 (whole segments) needs batch*H_kv <= %d CTAs (got %d)", grid, nseg);
  B200_REQUIRE(partition != 3 || csize > 1,
               "fused_decode_attention: partition 3 (a cluster per segment) needs batch*H_kv <= 64 (got %d)", nseg);
  p.partition = partition;
  p.gap = FD_GAP;
  p.cluster_size = csize;
  cudaError_t launched;
  if (csize > 1) {
    // every CTA of the launch must be resident together with its cluster mates; the other forms work with any grid
    int cgrid = cluster_limit(csize);
    if (cgrid > grid / csize * csize) cgrid = grid / csize * csize;
    launched = launch_pdl_cluster((overlap & OVERLAP_START) != 0, static_cast<unsigned>(csize), fused_decode_kernel,
                                  dim3(cgrid), dim3(FD_THREADS), FD_SMEM_TOTAL, reinterpret_cast<cudaStream_t>(stream), p,
                                  map_k, map_v);
  } else {
    launched = launch_pdl((overlap & OVERLAP_START) != 0, fused_decode_kernel, dim3(grid), dim3(FD_THREADS), FD_SMEM_TOTAL,
                          reinterpret_cast<cudaStream_t>(stream), p, map_k, map_v);
  }
  if (launched != cudaSuccess)
    return fail(ERR_LAUNCH, "fused_decode_attention: %s", cudaGetErrorString(cudaGetLastError()));
  return check_launch("fused_decode_attention");
}

// ---------------------------------------------------------------------------------------------------------------
// Variant for callers that cannot allocate device memory.
//
// Some hosts of this library hand out no allocator at all: a runtime that has already carved up the whole GPU and
// forbids cudaMalloc after start-up, a plugin loaded into somebody else's process that must not touch the caching
// allocator, or code running between the begin and end of a stream capture where an allocation is an error.  For
// them the fused decode step needs a workspace that exists without anyone asking for it.  It lives here, in a
// fixed-size array in the library's own device image: every GPU that loads the library carries these ~2 MB until the
// process exits, whether or not this entry point is ever called.
//
// The array's NAME is only meaningful to device code.  On the host the same identifier is a shadow object whose
// address is a host address, so it must never be handed to a kernel; the device address is asked for once per
// device with cudaGetSymbolAddress() while that device is current.
static __device__ __align__(256) unsigned char g_fused_decode_static_workspace[FD_WORKSPACE_BYTES];

static void* static_workspace_for_current_device() {
  static void* cached[64] = {nullptr};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (cached[dev] == nullptr) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_fused_decode_static_workspace) != cudaSuccess || ptr == nullptr) {
      cudaGetLastError();  // leave no sticky error behind for the caller's next launch check
      return nullptr;
    }
    cached[dev] = ptr;
  }
  return cached[dev];
}

extern "C" int b200_fused_decode_attention(const void* q, int64_t q_stride_b, int64_t q_stride_h, const void* k_new,
                                           int64_t kn_stride_b, int64_t kn_stride_h, const void* v_new,
                                           int64_t vn_stride_b, int64_t vn_stride_h, const void* gate,
                                           int64_t gate_stride_b, void* k_cache, void* v_cache, int64_t kc_stride_p,
                                           int64_t kc_stride_h, int64_t kc_stride_s, int64_t vc_stride_p,
                                           int64_t vc_stride_h, int64_t vc_stride_s, int64_t num_pages,
                                           const int32_t* block_table, int64_t bt_stride_b, const int64_t* pos,
                                           const float* inv_freq, int32_t rotary_dim, void* out, void* workspace,
                                           int32_t batch, int32_t num_q_heads, int32_t num_kv_heads, int32_t head_dim,
                                           b200_stream_t stream) {
  return fused_decode_impl(q, q_stride_b, q_stride_h, k_new, kn_stride_b, kn_stride_h, v_new, vn_stride_b, vn_stride_h,
                           gate, gate_stride_b, k_cache, v_cache, kc_stride_p, kc_stride_h, kc_stride_s, vc_stride_p,
                           vc_stride_h, vc_stride_s, num_pages, block_table, bt_stride_b, pos, inv_freq, rotary_dim, out,
                           workspace, batch, num_q_heads, num_kv_heads, head_dim, nullptr, nullptr, 0.f, 0, 0, stream);
}

extern "C" int b200_fused_decode_attention_ex(
    const void* q, int64_t q_stride_b, int64_t q_stride_h, const void* k_new, int64_t kn_stride_b, int64_t kn_stride_h,
    const void* v_new, int64_t vn_stride_b, int64_t vn_stride_h, const void* gate, int64_t gate_stride_b, void* k_cache,
    void* v_cache, int64_t kc_stride_p, int64_t kc_stride_h, int64_t kc_stride_s, int64_t vc_stride_p,
    int64_t vc_stride_h, int64_t vc_stride_s, int64_t num_pages, const int32_t* block_table, int64_t bt_stride_b,
    const int64_t* pos, const float* inv_freq, int32_t rotary_dim, void* out, void* workspace, int32_t batch,
    int32_t num_q_heads, int32_t num_kv_heads, int32_t head_dim, const void* q_norm_weight, const void* k_norm_weight,
    float eps, int32_t overlap, int32_t partition, b200_stream_t stream) {
  return fused_decode_impl(q, q_stride_b, q_stride_h, k_new, kn_stride_b, kn_stride_h, v_new, vn_stride_b, vn_stride_h,
                           gate, gate_stride_b, k_cache, v_cache, kc_stride_p, kc_stride_h, kc_stride_s, vc_stride_p,
                           vc_stride_h, vc_stride_s, num_pages, block_table, bt_stride_b, pos, inv_freq, rotary_dim, out,
                           workspace, batch, num_q_heads, num_kv_heads, head_dim, q_norm_weight, k_norm_weight, eps,
                           overlap, partition, stream);
}

// Same computation and arguments as b200_fused_decode_attention, minus the workspace.
//  - Nothing is allocated: no cudaMalloc / cudaFree, no allocating library call; the workspace is the static array.
//  - The FIRST call on each device looks up the array's device address (and raises the kernel's shared-memory
//    limit); make that first call outside any stream capture.  Later calls only enqueue work on `stream`.
//  - Limits (fixed by the array's size): batch <= 512 and batch * num_kv_heads <= 2048; larger calls are refused with
//    an error message and launch nothing.
//  - All calls on a device share the one array and it keeps what the previous call left in it.  The part that has
//    to start at zero (the per-segment arrival counters) is cleared on `stream` before each launch; the rest is
//    overwritten before it is read.  Two calls that overlap on the GPU (different streams, or graphs replayed
//    concurrently) would race on the array: serialise them.
extern "C" int b200_fused_decode_attention_static(const void* q, int64_t q_stride_b, int64_t q_stride_h,
                                                  const void* k_new, int64_t kn_stride_b, int64_t kn_stride_h,
                                                  const void* v_new, int64_t vn_stride_b, int64_t vn_stride_h,
                                                  const void* gate, int64_t gate_stride_b, void* k_cache,
                                                  void* v_cache, int64_t kc_stride_p, int64_t kc_stride_h,
                                                  int64_t kc_stride_s, int64_t vc_stride_p, int64_t vc_stride_h,
                                                  int64_t vc_stride_s, int64_t num_pages, const int32_t* block_table,
                                                  int64_t bt_stride_b, const int64_t* pos, const float* inv_freq,
                                                  int32_t rotary_dim, void* out, int32_t batch, int32_t num_q_heads,
                                                  int32_t num_kv_heads, int32_t head_dim, b200_stream_t stream) {
  if (batch < 1 || batch > FD_MAX_BATCH || num_kv_heads < 1 ||
      static_cast<int64_t>(batch) * num_kv_heads > FD_MAX_SEGMENTS)
    return fail(ERR_LIMIT,
                "fused_decode_attention_static: the built-in workspace holds at most batch=%d and batch*H_kv=%d "
                "(got batch=%d, H_kv=%d); use b200_fused_decode_attention with a caller-provided workspace",
                FD_MAX_BATCH, FD_MAX_SEGMENTS, batch, num_kv_heads);
  void* workspace = static_workspace_for_current_device();
  if (workspace == nullptr)
    return fail(ERR_RUNTIME, "fused_decode_attention_static: cudaGetSymbolAddress failed for the built-in workspace");
  if (cudaMemsetAsync(workspace, 0, FD_COUNTER_BYTES, reinterpret_cast<cudaStream_t>(stream)) != cudaSuccess)
    return fail(ERR_RUNTIME, "fused_decode_attention_static: cannot clear the arrival counters");
  return b200_fused_decode_attention(q, q_stride_b, q_stride_h, k_new, kn_stride_b, kn_stride_h, v_new, vn_stride_b,
                                     vn_stride_h, gate, gate_stride_b, k_cache, v_cache, kc_stride_p, kc_stride_h,
                                     kc_stride_s, vc_stride_p, vc_stride_h, vc_stride_s, num_pages, block_table,
                                     bt_stride_b, pos, inv_freq, rotary_dim, out, workspace, batch, num_q_heads,
                                     num_kv_heads, head_dim, stream);
}
