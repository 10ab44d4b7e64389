// Packed variable-length causal GQA prefill attention (4 Q heads per KV head, head_dim 256).
//   b200_fused_prefill_attention  <-> the chain of engine/runner.py:339-384: partial_rope(q), partial_rope(k),
//                                     gqa_attention_varlen_causal, attention_gate_pack, paged_kv_fill_varlen
//
// One CTA = one (sequence, kv head, block of 32 query rows): the 4 Q heads of the group are stacked, so each
// K/V tile is fetched once per group (the stacking of gqa_attention_varlen_causal.py:151-160).  8 warps, warp w
// owns head (w & 3) and the 16-row half (w >> 2).  K/V tiles of 64 tokens are staged by the TMA engine as one
// 512-byte bulk copy per token row at a 528-byte pitch (conflict-free ldmatrix), double buffered on mbarriers.
// The rows come either from the packed [T, H_kv, D] tensors (drop-in operator) or from the paged cache through
// the page table (fused path: a first small kernel rotates K and scatters K/V into the cache, the attention
// kernel then reads the cache, so the rotation is computed once per token instead of once per consumer tile).
// Arithmetic mirrors the reference: q is scaled by scale*log2(e) and RE-ROUNDED to bf16 before QK^T, exp2
// softmax, p rounded to bf16 for PV while l sums the fp32 p, acc / l rounded to bf16.
#include "b200_attn.h"
#include "common.cuh"

namespace b200 {

constexpr int PF_BQ = 32;                    // query rows per CTA (per head)
constexpr int PF_TKV = 64;                   // KV tokens per tile
constexpr int PF_WARPS = 8;
constexpr int PF_THREADS = PF_WARPS * 32;
constexpr int PF_PITCH = HEAD_DIM * 2 + 16;  // 528-byte row pitch in shared memory
constexpr int PF_Q_BYTES = GROUP * PF_BQ * PF_PITCH;   // 128 rows
constexpr int PF_KV_BYTES = PF_TKV * PF_PITCH;          // one K (or V) tile
constexpr int PF_SMEM = PF_Q_BYTES + 4 * PF_KV_BYTES + 128;
constexpr float LOG2E = 1.4426950408889634f;

struct PrefillParams {
  const __nv_bfloat16 *q, *k, *v, *gate;
  __nv_bfloat16* out;
  int64_t q_t, q_h, k_t, k_h, v_t, v_h, out_t, out_h, gate_t;
  // paged source (fused path)
  const __nv_bfloat16 *k_cache, *v_cache;
  int64_t kc_p, kc_h, kc_s, vc_p, vc_h, vc_s, bt_b;
  const int32_t* block_table;
  const int32_t* cu_seqlens;
  const void* position_ids;  // [T] int32 or int64 (fused path: rope on q)
  int ids_are_int64;
  const float* inv_freq;
  int* err;
  float qk_scale;
};

template <bool PAGED, bool FUSED>
__global__ void __launch_bounds__(PF_THREADS, 1) varlen_causal_kernel(const __grid_constant__ PrefillParams p) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  __shared__ uint64_t bar_q, bar_kv[2];
  __shared__ float rope_cs[FUSED ? PF_BQ * 32 * 2 : 2];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
  uint8_t* q_s = smem;
  uint8_t* kv_s = smem + PF_Q_BYTES;  // [stage][K | V]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int qb = gridDim.x - 1 - blockIdx.x;  // heaviest blocks first
  const int h = blockIdx.y, b = blockIdx.z;
  const int seq_start = p.cu_seqlens[b];
  const int seq_len = p.cu_seqlens[b + 1] - seq_start;
  const int q0 = qb * PF_BQ;
  if (q0 >= seq_len) return;

  if (tid == 0) {
    mbar_init(&bar_q, 1);
    mbar_init(&bar_kv[0], 1);
    mbar_init(&bar_kv[1], 1);
    mbar_fence_init();
  }
  __syncthreads();

  const int kv_end = min(q0 + PF_BQ, seq_len);
  const int n_tiles = (kv_end + PF_TKV - 1) / PF_TKV;

  auto issue_tile = [&](int tile) {
    // threads 0..63 copy K rows, 64..127 copy V rows; rows past the end repeat the last valid token (finite
    // data that the mask removes)
    const int stage = tile & 1;
    if (tid == 0) mbar_expect_tx(&bar_kv[stage], 2 * PF_TKV * HEAD_DIM * 2);
    if (tid < 2 * PF_TKV) {
      const int r = tid & (PF_TKV - 1);
      const bool is_v = tid >= PF_TKV;
      const int tok = min(tile * PF_TKV + r, seq_len - 1);
      const __nv_bfloat16* src;
      if (PAGED) {
        const int64_t phys = p.block_table[b * p.bt_b + tok / PAGE];
        src = is_v ? p.v_cache + phys * p.vc_p + h * p.vc_h + (tok % PAGE) * p.vc_s
                   : p.k_cache + phys * p.kc_p + h * p.kc_h + (tok % PAGE) * p.kc_s;
      } else {
        src = is_v ? p.v + static_cast<int64_t>(seq_start + tok) * p.v_t + h * p.v_h
                   : p.k + static_cast<int64_t>(seq_start + tok) * p.k_t + h * p.k_h;
      }
      uint8_t* dst = kv_s + (stage * 2 + (is_v ? 1 : 0)) * PF_KV_BYTES + r * PF_PITCH;
      bulk_g2s(dst, src, HEAD_DIM * 2, &bar_kv[stage]);
    }
  };

  // ---- Q tile: 4 heads x 32 rows, row index = head * 32 + r
  if (tid == 0) mbar_expect_tx(&bar_q, GROUP * PF_BQ * HEAD_DIM * 2);
  __syncthreads();  // expect_tx registered before any copy can complete the phase
  if (tid < GROUP * PF_BQ) {
    const int hh = tid / PF_BQ, r = tid % PF_BQ;
    const int row = min(q0 + r, seq_len - 1);
    bulk_g2s(q_s + tid * PF_PITCH, p.q + static_cast<int64_t>(seq_start + row) * p.q_t + (h * GROUP + hh) * p.q_h,
             HEAD_DIM * 2, &bar_q);
  }
  issue_tile(0);
  if (n_tiles > 1) issue_tile(1);

  if (FUSED) {
    // cos/sin of the 32 query rows x 32 rotary pairs, shared by the 4 heads
    for (int i = tid; i < PF_BQ * 32; i += PF_THREADS) {
      const int r = i >> 5, j = i & 31;
      const int64_t t = seq_start + min(q0 + r, seq_len - 1);
      const int64_t pid = p.ids_are_int64 ? static_cast<const int64_t*>(p.position_ids)[t]
                                          : static_cast<int64_t>(static_cast<const int32_t*>(p.position_ids)[t]);
      float sn, cs;
      sincosf(static_cast<float>(pid) * p.inv_freq[j], &sn, &cs);
      rope_cs[i * 2] = cs;
      rope_cs[i * 2 + 1] = sn;
    }
  }
  bool ok = mbar_wait_bounded(&bar_q, 0);
  __syncthreads();
  // ---- in place: (rope) -> * scale*log2(e) -> bf16
  if (FUSED) {
    for (int i = tid; i < GROUP * PF_BQ * 32; i += PF_THREADS) {
      const int row = i >> 5, j = i & 31, r = row % PF_BQ;
      __nv_bfloat16* qr = reinterpret_cast<__nv_bfloat16*>(q_s + row * PF_PITCH);
      const float cs = rope_cs[(r * 32 + j) * 2], sn = rope_cs[(r * 32 + j) * 2 + 1];
      float f, g;
      rope_pair(__bfloat162float(qr[j]), __bfloat162float(qr[j + 32]), sn, cs, f, g);
      qr[j] = __float2bfloat16_rn(f);
      qr[j + 32] = __float2bfloat16_rn(g);
    }
    __syncthreads();
  }
  for (int i = tid; i < GROUP * PF_BQ * (HEAD_DIM / 8); i += PF_THREADS) {
    const int row = i / (HEAD_DIM / 8), c = i % (HEAD_DIM / 8);
    uint4* ptr = reinterpret_cast<uint4*>(q_s + row * PF_PITCH + c * 16);
    uint4 v = *ptr;
    uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) w[j] = pack_bf16(bf16_lo(w[j]) * p.qk_scale, bf16_hi(w[j]) * p.qk_scale);
    *ptr = make_uint4(w[0], w[1], w[2], w[3]);
  }
  __syncthreads();

  const int hh = warp & 3, rh = warp >> 2;
  const uint32_t q_base = smem_u32(q_s) + (hh * PF_BQ + rh * 16) * PF_PITCH;
  const int mi = lane >> 3, r8 = lane & 7;
  const uint32_t q_addr = q_base + (r8 + (mi & 1) * 8) * PF_PITCH + (mi >> 1) * 16;
  const int row0 = q0 + rh * 16 + (lane >> 2);  // sequence-local query index of c[0], c[1]; +8 for c[2], c[3]

  float o[32][4];
#pragma unroll
  for (int i = 0; i < 32; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

  for (int tile = 0; tile < n_tiles; ++tile) {
    const int stage = tile & 1;
    if (ok) ok = mbar_wait_bounded(&bar_kv[stage], (tile >> 1) & 1);
    const uint32_t k_base = smem_u32(kv_s + (stage * 2) * PF_KV_BYTES);
    const uint32_t v_base = k_base + PF_KV_BYTES;
    const int t0 = tile * PF_TKV;
    if (ok) {
      // ---- S = Q K^T : [16 x 64] per warp
      float s[8][4];
#pragma unroll
      for (int i = 0; i < 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
      const uint32_t k_addr = k_base + ((mi >> 1) * 8 + r8) * PF_PITCH + (mi & 1) * 16;
#pragma unroll 4
      for (int ks = 0; ks < 16; ++ks) {
        uint32_t a[4];
        ldmatrix_x4(a, q_addr + ks * 32);
#pragma unroll
        for (int np = 0; np < 4; ++np) {
          uint32_t bk[4];
          ldmatrix_x4(bk, k_addr + np * 16 * PF_PITCH + ks * 32);
          mma_bf16_16816(s[2 * np], a, bk[0], bk[1]);
          mma_bf16_16816(s[2 * np + 1], a, bk[2], bk[3]);
        }
      }
      // ---- mask: causal and inside the sequence (only tiles that touch the diagonal or the end need it)
      if (t0 + PF_TKV - 1 > q0 + rh * 16 || t0 + PF_TKV > seq_len) {
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
          const int c0 = t0 + nt * 8 + (lane & 3) * 2;
          if (!(c0 <= row0 && c0 < seq_len)) s[nt][0] = -INFINITY;
          if (!(c0 + 1 <= row0 && c0 + 1 < seq_len)) s[nt][1] = -INFINITY;
          if (!(c0 <= row0 + 8 && c0 < seq_len)) s[nt][2] = -INFINITY;
          if (!(c0 + 1 <= row0 + 8 && c0 + 1 < seq_len)) s[nt][3] = -INFINITY;
        }
      }
      // ---- online softmax (base 2), rows lane>>2 and +8, reduced over the 4 lanes of a quad
      float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        mx0 = fmaxf(mx0, fmaxf(s[nt][0], s[nt][1]));
        mx1 = fmaxf(mx1, fmaxf(s[nt][2], s[nt][3]));
      }
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      const float m0 = fmaxf(m_run[0], mx0), m1 = fmaxf(m_run[1], mx1);
      // a row whose every column so far is masked keeps m = -inf: use 0 as the subtrahend so exp2 sees -inf, not NaN
      const float sub0 = (m0 == -INFINITY) ? 0.f : m0, sub1 = (m1 == -INFINITY) ? 0.f : m1;
      const float alpha0 = exp2f(m_run[0] - sub0), alpha1 = exp2f(m_run[1] - sub1);
      float sum0 = 0.f, sum1 = 0.f;
      uint32_t pa[4][4];
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        const float p0 = exp2f(s[nt][0] - sub0), p1 = exp2f(s[nt][1] - sub0);
        const float p2 = exp2f(s[nt][2] - sub1), p3 = exp2f(s[nt][3] - sub1);
        sum0 += p0 + p1;
        sum1 += p2 + p3;
        pa[nt >> 1][(nt & 1) * 2] = pack_bf16(p0, p1);
        pa[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16(p2, p3);
      }
      sum0 += __shfl_xor_sync(0xffffffffu, sum0, 1);
      sum0 += __shfl_xor_sync(0xffffffffu, sum0, 2);
      sum1 += __shfl_xor_sync(0xffffffffu, sum1, 1);
      sum1 += __shfl_xor_sync(0xffffffffu, sum1, 2);
      l_run[0] = l_run[0] * alpha0 + sum0;
      l_run[1] = l_run[1] * alpha1 + sum1;
      m_run[0] = m0;
      m_run[1] = m1;
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        o[i][0] *= alpha0;
        o[i][1] *= alpha0;
        o[i][2] *= alpha1;
        o[i][3] *= alpha1;
      }
      // ---- O += P V
      const uint32_t v_addr = v_base + ((mi & 1) * 8 + r8) * PF_PITCH + (mi >> 1) * 16;
#pragma unroll
      for (int kt = 0; kt < 4; ++kt) {
#pragma unroll
        for (int dp = 0; dp < 16; ++dp) {
          uint32_t bv[4];
          ldmatrix_x4_trans(bv, v_addr + kt * 16 * PF_PITCH + dp * 32);
          mma_bf16_16816(o[2 * dp], pa[kt], bv[0], bv[1]);
          mma_bf16_16816(o[2 * dp + 1], pa[kt], bv[2], bv[3]);
        }
      }
    }
    __syncthreads();  // every warp is done with this stage
    if (tile + 2 < n_tiles) issue_tile(tile + 2);
  }
  if (!ok) {
    if (tid == 0) atomicExch(p.err, 1);
    // give copies still in flight a bounded time to land before the CTA's shared memory is released
    mbar_wait_bounded(&bar_q, 0, 1u << 12);
    return;
  }

  // ---- epilogue: acc / l -> bf16 into this warp's own Q rows (free now), then 16-byte coalesced stores
  __syncwarp();
  {
    const float inv0 = 1.f / l_run[0], inv1 = 1.f / l_run[1];
    uint8_t* my_rows = q_s + (hh * PF_BQ + rh * 16) * PF_PITCH;
    const int r = lane >> 2, c = (lane & 3) * 2;
#pragma unroll
    for (int nt = 0; nt < 32; ++nt) {
      *reinterpret_cast<uint32_t*>(my_rows + r * PF_PITCH + (nt * 8 + c) * 2) = pack_bf16(o[nt][0] * inv0, o[nt][1] * inv0);
      *reinterpret_cast<uint32_t*>(my_rows + (r + 8) * PF_PITCH + (nt * 8 + c) * 2) =
          pack_bf16(o[nt][2] * inv1, o[nt][3] * inv1);
    }
    __syncwarp();
    for (int i = lane; i < 16 * (HEAD_DIM / 8); i += 32) {
      const int rr = i / (HEAD_DIM / 8), cc = i % (HEAD_DIM / 8);
      const int row = q0 + rh * 16 + rr;
      if (row < seq_len) {
        uint4 v = *reinterpret_cast<const uint4*>(my_rows + rr * PF_PITCH + cc * 16);
        const int64_t t = seq_start + row;
        if (FUSED) {
          const uint4 gv = *reinterpret_cast<const uint4*>(p.gate + t * p.gate_t + (h * GROUP + hh) * HEAD_DIM + cc * 8);
          uint32_t xs[4] = {v.x, v.y, v.z, v.w};
          const uint32_t gs[4] = {gv.x, gv.y, gv.z, gv.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float g0 = 1.f / (1.f + __expf(-bf16_lo(gs[j]))), g1 = 1.f / (1.f + __expf(-bf16_hi(gs[j])));
            xs[j] = pack_bf16(bf16_lo(xs[j]) * g0, bf16_hi(xs[j]) * g1);
          }
          v = make_uint4(xs[0], xs[1], xs[2], xs[3]);
        }
        *reinterpret_cast<uint4*>(p.out + t * p.out_t + (h * GROUP + hh) * p.out_h + cc * 8) = v;
      }
    }
  }
}

// Fused path, first kernel: rotate K at its position and scatter K (rotated) and V into the paged cache.
// One warp per (token, kv head) row, each lane 8 consecutive dims; grid = (pages of the longest sequence, H_kv, B).
__global__ void __launch_bounds__(128)
rope_scatter_kernel(const __nv_bfloat16* __restrict__ k, int64_t k_t, int64_t k_h, const __nv_bfloat16* __restrict__ v,
                    int64_t v_t, int64_t v_h, __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache,
                    int64_t kc_p, int64_t kc_h, int64_t kc_s, int64_t vc_p, int64_t vc_h, int64_t vc_s,
                    const int32_t* __restrict__ block_table, int64_t bt_b, const int32_t* __restrict__ cu_seqlens,
                    const void* __restrict__ position_ids, int ids_are_int64, const float* __restrict__ inv_freq,
                    int rotary_half) {
  const int lp = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int seq_start = cu_seqlens[b];
  const int seq_len = cu_seqlens[b + 1] - seq_start;
  if (lp * PAGE >= seq_len) return;
  const int64_t phys = block_table[b * bt_b + lp];
  const int lanes_half = rotary_half / 8;
  const bool in_rot = lane < 2 * lanes_half;
  const bool first = lane < lanes_half;
  const int partner = first ? lane + lanes_half : lane - lanes_half;
  for (int slot = warp; slot < PAGE; slot += 4) {
    const int tok = lp * PAGE + slot;
    if (tok >= seq_len) break;
    const int64_t t = seq_start + tok;
    const uint4 kraw = *reinterpret_cast<const uint4*>(k + t * k_t + h * k_h + lane * 8);
    const uint4 vraw = *reinterpret_cast<const uint4*>(v + t * v_t + h * v_h + lane * 8);
    uint32_t kw[4] = {kraw.x, kraw.y, kraw.z, kraw.w};
    if (rotary_half > 0) {
      uint32_t other[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) other[i] = __shfl_sync(0xffffffffu, kw[i], in_rot ? partner : lane);
      if (in_rot) {
        const int64_t pid = ids_are_int64 ? static_cast<const int64_t*>(position_ids)[t]
                                          : static_cast<int64_t>(static_cast<const int32_t*>(position_ids)[t]);
        const float posf = static_cast<float>(pid);
        const int dbase = (first ? lane : partner) * 8;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float s0, c0, s1, c1;
          sincosf(posf * inv_freq[dbase + 2 * i], &s0, &c0);
          sincosf(posf * inv_freq[dbase + 2 * i + 1], &s1, &c1);
          const uint32_t fa = first ? kw[i] : other[i];
          const uint32_t fb = first ? other[i] : kw[i];
          float f0, g0, f1, g1;
          rope_pair(bf16_lo(fa), bf16_lo(fb), s0, c0, f0, g0);
          rope_pair(bf16_hi(fa), bf16_hi(fb), s1, c1, f1, g1);
          kw[i] = first ? pack_bf16(f0, f1) : pack_bf16(g0, g1);
        }
      }
    }
    *reinterpret_cast<uint4*>(k_cache + phys * kc_p + h * kc_h + slot * kc_s + lane * 8) = make_uint4(kw[0], kw[1], kw[2], kw[3]);
    *reinterpret_cast<uint4*>(v_cache + phys * vc_p + h * vc_h + slot * vc_s + lane * 8) = vraw;
  }
}

template <bool PAGED, bool FUSED>
static int launch_varlen(const PrefillParams& p, int batch, int num_kv_heads, int max_seqlen, cudaStream_t stream) {
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    if (cudaFuncSetAttribute(varlen_causal_kernel<PAGED, FUSED>, cudaFuncAttributeMaxDynamicSharedMemorySize, PF_SMEM) !=
        cudaSuccess)
      return fail(ERR_RUNTIME, "varlen attention: cannot raise dynamic shared memory to %d", PF_SMEM);
    configured[dev] = true;
  }
  const dim3 grid((max_seqlen + PF_BQ - 1) / PF_BQ, num_kv_heads, batch);
  varlen_causal_kernel<PAGED, FUSED><<<grid, PF_THREADS, PF_SMEM, stream>>>(p);
  return check_launch("varlen attention");
}

}  // namespace b200

using namespace b200;

static bool mult8(int64_t x) { return (x & 7) == 0; }

extern "C" int b200_fused_prefill_attention(const void* q, int64_t q_stride_t, int64_t q_stride_h, const void* k,
                                            int64_t k_stride_t, int64_t k_stride_h, const void* v, int64_t v_stride_t,
                                            int64_t v_stride_h, const void* gate, int64_t gate_stride_t, void* k_cache,
                                            void* v_cache, int64_t kc_stride_p, int64_t kc_stride_h,
                                            int64_t kc_stride_s, int64_t vc_stride_p, int64_t vc_stride_h,
                                            int64_t vc_stride_s, const int32_t* block_table, int64_t bt_stride_b,
                                            const int32_t* cu_seqlens, const void* position_ids, int32_t ids_are_int64,
                                            const float* inv_freq, int32_t rotary_dim, void* out, int32_t batch,
                                            int32_t max_seqlen, int32_t num_q_heads, int32_t num_kv_heads,
                                            int32_t head_dim, b200_stream_t stream) {
  B200_REQUIRE(batch > 0 && batch <= 65535, "fused_prefill_attention: batch must be in [1, 65535]");
  B200_REQUIRE(head_dim == HEAD_DIM, "fused_prefill_attention: head_dim must be %d (got %d)", HEAD_DIM, head_dim);
  B200_REQUIRE(num_kv_heads > 0 && num_q_heads == num_kv_heads * GROUP,
               "fused_prefill_attention: needs %d Q heads per KV head (got %d/%d)", GROUP, num_q_heads, num_kv_heads);
  B200_REQUIRE(rotary_dim == 64, "fused_prefill_attention: rotary_dim must be 64 (got %d)", rotary_dim);
  B200_REQUIRE(inv_freq != nullptr && position_ids != nullptr, "fused_prefill_attention: NULL rope inputs");
  B200_REQUIRE(aligned16(q) && aligned16(k) && aligned16(v) && aligned16(out) && aligned16(gate) &&
                   aligned16(k_cache) && aligned16(v_cache) && mult8(q_stride_t) && mult8(q_stride_h) &&
                   mult8(k_stride_t) && mult8(k_stride_h) && mult8(v_stride_t) && mult8(v_stride_h) &&
                   mult8(gate_stride_t) && mult8(kc_stride_p) && mult8(kc_stride_h) && mult8(kc_stride_s) &&
                   mult8(vc_stride_p) && mult8(vc_stride_h) && mult8(vc_stride_s),
               "fused_prefill_attention: tensors must be 16-byte aligned with strides that are multiples of 8");
  if (max_seqlen <= 0) return OK;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const dim3 grid((max_seqlen + PAGE - 1) / PAGE, num_kv_heads, batch);
  rope_scatter_kernel<<<grid, 128, 0, st>>>(
      static_cast<const __nv_bfloat16*>(k), k_stride_t, k_stride_h, static_cast<const __nv_bfloat16*>(v), v_stride_t,
      v_stride_h, static_cast<__nv_bfloat16*>(k_cache), static_cast<__nv_bfloat16*>(v_cache), kc_stride_p, kc_stride_h,
      kc_stride_s, vc_stride_p, vc_stride_h, vc_stride_s, block_table, bt_stride_b, cu_seqlens, position_ids,
      ids_are_int64, inv_freq, rotary_dim / 2);
  int rc = check_launch("fused_prefill_attention (rope + scatter)");
  if (rc != OK) return rc;
  PrefillParams p = {};
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.gate = static_cast<const __nv_bfloat16*>(gate);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.q_t = q_stride_t; p.q_h = q_stride_h;
  p.out_t = static_cast<int64_t>(num_q_heads) * HEAD_DIM; p.out_h = HEAD_DIM;
  p.gate_t = gate_stride_t;
  p.k_cache = static_cast<const __nv_bfloat16*>(k_cache);
  p.v_cache = static_cast<const __nv_bfloat16*>(v_cache);
  p.kc_p = kc_stride_p; p.kc_h = kc_stride_h; p.kc_s = kc_stride_s;
  p.vc_p = vc_stride_p; p.vc_h = vc_stride_h; p.vc_s = vc_stride_s;
  p.bt_b = bt_stride_b;
  p.block_table = block_table;
  p.cu_seqlens = cu_seqlens;
  p.position_ids = position_ids;
  p.ids_are_int64 = ids_are_int64;
  p.inv_freq = inv_freq;
  p.err = wait_timeout_flag();
  if (!p.err) return fail(ERR_RUNTIME, "fused_prefill_attention: no error flag");
  p.qk_scale = (1.0f / sqrtf(static_cast<float>(head_dim))) * LOG2E;
  return launch_varlen<true, true>(p, batch, num_kv_heads, max_seqlen, st);
}
