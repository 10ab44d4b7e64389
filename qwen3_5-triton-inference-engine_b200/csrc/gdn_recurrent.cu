// Gated-DeltaNet delta-rule recurrence, token-serial forms (fp32 state [128 x 128] per head):
//   b200_gdn_recurrent_decode              <-> triton_kernels/gdn_recurrent_prefill.py:145-246 (+ op :1185-1259)
//   b200_gdn_recurrent_prefill_sequential  <-> triton_kernels/gdn_recurrent_prefill.py:47-143  (+ op :1050-1145)
// Per token:  S *= exp(g);  mem = k^T S;  delta = beta (v - mem);  S += k (x) delta;  out = q^T S.
//
// Layout: one CTA per (sequence, head), one thread per value column.  A thread keeps its whole column
// S[0..127][v] in registers, so both column reductions (k^T S and q^T S) are thread-local: no shuffles and
// no block barriers inside a token.  Global accesses are coalesced along v (a warp touches 128 contiguous
// bytes per state row).  Decode streams the 64 KiB state once in and once out (HBM-bound); prefill keeps it
// in registers across the whole sequence (fp32-FMA-bound).
//
// Decode exists in three forms, chosen by size (measured on B200, fractions of the measured copy bandwidth):
//   * gdn_decode_slice_kernel: CTA = one warp = 32 columns of one head, the column in registers.  Best for very many
//     heads (4096 heads: 0.99) and in the gap around one to three heads per SM.
//   * gdn_decode_ring_kernel: persistent CTAs with a ring of [128 x 16] boxes moved by tensor-map TMA and a copy warp.
//     Best (or level) from one head up to about two thousand (512 heads: 0.78, 1024: 0.88, 2048: 0.94): several small
//     rings per SM stagger the load, update and store phases that one wave of register-resident heads runs in lockstep.
//     Needs the dense [B, H, 128, 128] state.
//   * gdn_decode_kernel: CTA = one head, any strides and alignments; the fallback.
#include "b200_attn.h"
#include "umma.cuh"

#include <atomic>

namespace b200 {

constexpr int GDN_THREADS = GDN_D;  // one thread per value column

// k and q of one token as fp32 in shared memory, read back as broadcast float4.
__device__ __forceinline__ void gdn_token_update(float (&s)[GDN_D], const float* __restrict__ kf,
                                                 const float* __restrict__ qf, float eg, float beta, float v,
                                                 float& out) {
  float mem0 = 0.f, mem1 = 0.f, mem2 = 0.f, mem3 = 0.f;
#pragma unroll
  for (int i = 0; i < GDN_D; i += 4) {
    const float4 k4 = *reinterpret_cast<const float4*>(kf + i);
    s[i] *= eg;
    s[i + 1] *= eg;
    s[i + 2] *= eg;
    s[i + 3] *= eg;
    mem0 = fmaf(k4.x, s[i], mem0);
    mem1 = fmaf(k4.y, s[i + 1], mem1);
    mem2 = fmaf(k4.z, s[i + 2], mem2);
    mem3 = fmaf(k4.w, s[i + 3], mem3);
  }
  const float delta = beta * (v - ((mem0 + mem1) + (mem2 + mem3)));
  float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
  for (int i = 0; i < GDN_D; i += 4) {
    const float4 k4 = *reinterpret_cast<const float4*>(kf + i);
    const float4 q4 = *reinterpret_cast<const float4*>(qf + i);
    s[i] = fmaf(k4.x, delta, s[i]);
    s[i + 1] = fmaf(k4.y, delta, s[i + 1]);
    s[i + 2] = fmaf(k4.z, delta, s[i + 2]);
    s[i + 3] = fmaf(k4.w, delta, s[i + 3]);
    o0 = fmaf(q4.x, s[i], o0);
    o1 = fmaf(q4.y, s[i + 1], o1);
    o2 = fmaf(q4.z, s[i + 2], o2);
    o3 = fmaf(q4.w, s[i + 3], o3);
  }
  out = (o0 + o1) + (o2 + o3);
}

__global__ void __launch_bounds__(GDN_THREADS)
gdn_decode_kernel(const __nv_bfloat16* q, int64_t q_b, int64_t q_h, const __nv_bfloat16* k,
                  int64_t k_b, int64_t k_h, const __nv_bfloat16* v, int64_t v_b, int64_t v_h,
                  const float* beta, int64_t be_b, int64_t be_h, const float* g, int64_t g_b,
                  int64_t g_h, float* state, int64_t s_b, int64_t s_h, __nv_bfloat16* out,
                  int64_t o_b, int64_t o_h, int heads) {
  pdl_chain();
  __shared__ __align__(16) float kf[GDN_D];
  __shared__ __align__(16) float qf[GDN_D];
  const int b = blockIdx.x / heads, h = blockIdx.x % heads, col = threadIdx.x;
  float* sp = state + b * s_b + h * s_h + col;
  float s[GDN_D];
#pragma unroll
  for (int i = 0; i < GDN_D; ++i) s[i] = __ldcs(sp + i * GDN_D);  // streamed once: evict-first
  kf[col] = __bfloat162float(k[b * k_b + h * k_h + col]);
  qf[col] = __bfloat162float(q[b * q_b + h * q_h + col]);
  const float eg = __expf(g[b * g_b + h * g_h]);
  const float bt = beta[b * be_b + h * be_h];
  const float vv = __bfloat162float(v[b * v_b + h * v_h + col]);
  __syncthreads();
  float o;
  gdn_token_update(s, kf, qf, eg, bt, vv, o);
  out[b * o_b + h * o_h + col] = __float2bfloat16_rn(o);
#pragma unroll
  for (int i = 0; i < GDN_D; ++i) __stcs(sp + i * GDN_D, s[i]);
}

// The same step with a finer grain: CTA = ONE warp = 32 value columns of one (sequence, head).  Four times as many, four
// times smaller work items than gdn_decode_kernel (eight resident per SM: the same two heads of state in registers,
// but they retire and start a quarter head at a time), so the SMs stay evenly loaded and the last wave is a
// quarter as long.  Used while the batch is too small to keep every SM busy for several rounds with whole heads.
constexpr int GDN_SLICE = 32;

__global__ void __launch_bounds__(GDN_SLICE, 8)
gdn_decode_slice_kernel(const __nv_bfloat16* q, int64_t q_b, int64_t q_h, const __nv_bfloat16* k,
                        int64_t k_b, int64_t k_h, const __nv_bfloat16* v, int64_t v_b, int64_t v_h,
                        const float* beta, int64_t be_b, int64_t be_h, const float* g,
                        int64_t g_b, int64_t g_h, float* state, int64_t s_b, int64_t s_h,
                        __nv_bfloat16* out, int64_t o_b, int64_t o_h, int heads) {
  pdl_chain();
  __shared__ __align__(16) float kf[GDN_D];
  __shared__ __align__(16) float qf[GDN_D];
  constexpr int SLICES = GDN_D / GDN_SLICE;
  const int item = blockIdx.x / SLICES, slice = blockIdx.x % SLICES;
  const int b = item / heads, h = item % heads, lane = threadIdx.x, col = slice * GDN_SLICE + lane;
  float* sp = state + b * s_b + h * s_h + col;
  // k and q of the head: 4 values per lane, widened into shared memory for the broadcast reads of the update
  {
    const uint2 kr = *reinterpret_cast<const uint2*>(k + b * k_b + h * k_h + lane * 4);
    const uint2 qr = *reinterpret_cast<const uint2*>(q + b * q_b + h * q_h + lane * 4);
    *reinterpret_cast<float4*>(kf + lane * 4) = make_float4(bf16_lo(kr.x), bf16_hi(kr.x), bf16_lo(kr.y), bf16_hi(kr.y));
    *reinterpret_cast<float4*>(qf + lane * 4) = make_float4(bf16_lo(qr.x), bf16_hi(qr.x), bf16_lo(qr.y), bf16_hi(qr.y));
  }
  const float eg = __expf(g[b * g_b + h * g_h]);
  const float bt = beta[b * be_b + h * be_h];
  const float vv = __bfloat162float(v[b * v_b + h * v_h + col]);
  float s[GDN_D];
#pragma unroll
  for (int i = 0; i < GDN_D; ++i) s[i] = __ldcs(sp + i * GDN_D);  // streamed once: evict-first
  __syncwarp();
  float o;
  gdn_token_update(s, kf, qf, eg, bt, vv, o);
  out[b * o_b + h * o_h + col] = __float2bfloat16_rn(o);
#pragma unroll
  for (int i = 0; i < GDN_D; ++i) __stcs(sp + i * GDN_D, s[i]);
}

// The whole Gated-DeltaNet mixer of one decode token between its two projections, in one launch per layer:
// conv state shift + depthwise conv4 + SiLU (triton_kernels/depthwise_causal_conv4_decode.py), q/k L2 norms and the
// beta / g gates (triton_kernels/gdn_qk_norm_gates.py:68-89), the delta-rule step above, and the gated RMSNorm
// (triton_kernels/gdn_gated_rmsnorm.py:54-67).  `fused` is one row of the input projection per sequence:
// [q | k | v | z | a | b] = [3*H*128 | H*128 | H | H].  Thread t of CTA (sequence, head) owns channel t of the head's q,
// k, v and z slices and value column t of the state; every intermediate keeps the reference's rounding point (conv
// output, q_n, k_n and the recurrence output are bf16 tensors there).
__global__ void __launch_bounds__(GDN_THREADS)
gdn_decode_fused_kernel(const __nv_bfloat16* fused, int64_t fused_stride,  // no __restrict__: see pdl_wait()
                        __nv_bfloat16* __restrict__ conv_state, const __nv_bfloat16* __restrict__ w4,
                        const float* __restrict__ a_log, const __nv_bfloat16* __restrict__ dt_bias,
                        const float* __restrict__ norm_w, float* __restrict__ state, __nv_bfloat16* __restrict__ out,
                        int heads, int overlap) {
  __shared__ __align__(16) float kf[GDN_D];
  __shared__ __align__(16) float qf[GDN_D];
  __shared__ float red[3][4];
  __shared__ float gate_s[2];
  const int b = blockIdx.x / heads, h = blockIdx.x % heads, t = threadIdx.x;
  const int kd = heads * GDN_D, width = 3 * kd;
  float* sp = state + (static_cast<int64_t>(b) * heads + h) * GDN_D * GDN_D + t;
  const __nv_bfloat16* row = fused + static_cast<int64_t>(b) * fused_stride;
  // With the PREFETCH flag the caller guarantees that the conv state and the recurrent state were last written by an
  // EARLIER kernel than the one directly before this one in the stream (in a layer stack that one is the input
  // projection): their loads then go out before pdl_wait() and overlap with the projection.  `fused` is read after
  // the wait; every store comes after it too.
  if (overlap & OVERLAP_TRIGGER) pdl_trigger();
  if (!(overlap & OVERLAP_PREFETCH)) pdl_wait();
  __nv_bfloat16 cs[3][3], cx[3], cw[3][4];
#pragma unroll
  for (int part = 0; part < 3; ++part) {
    const int c = part * kd + h * GDN_D + t;
    const __nv_bfloat16* st = conv_state + static_cast<int64_t>(b) * 4 * width + c;
    cs[part][0] = st[width];
    cs[part][1] = st[2 * width];
    cs[part][2] = st[3 * width];
#pragma unroll
    for (int r = 0; r < 4; ++r) cw[part][r] = w4[r * width + c];
  }
  // the weights of the epilogue and of the gates are fetched up front as well: nothing later waits for a first touch
  const float wv = norm_w[t];
  const float a_log_h = a_log[h], dt_bias_h = __bfloat162float(dt_bias[h]);
  float s[GDN_D];
#pragma unroll
  for (int i = 0; i < GDN_D; ++i) s[i] = __ldcs(sp + i * GDN_D);  // streamed once: evict-first
  pdl_wait();
  // every value of the projection row this thread needs, in one round trip
#pragma unroll
  for (int part = 0; part < 3; ++part) cx[part] = row[part * kd + h * GDN_D + t];
  const float zv = __bfloat162float(row[width + h * GDN_D + t]);
  const float a_raw = __bfloat162float(row[width + kd + h]), b_raw = __bfloat162float(row[width + kd + heads + h]);
  float y[3];
#pragma unroll
  for (int part = 0; part < 3; ++part) {
    const int c = part * kd + h * GDN_D + t;
    __nv_bfloat16* st = conv_state + static_cast<int64_t>(b) * 4 * width + c;
    st[0] = cs[part][0];
    st[width] = cs[part][1];
    st[2 * width] = cs[part][2];
    st[3 * width] = cx[part];
    float acc = __bfloat162float(cw[part][0]) * __bfloat162float(cs[part][0]);
    acc = fmaf(__bfloat162float(cw[part][1]), __bfloat162float(cs[part][1]), acc);
    acc = fmaf(__bfloat162float(cw[part][2]), __bfloat162float(cs[part][2]), acc);
    acc = fmaf(__bfloat162float(cw[part][3]), __bfloat162float(cx[part]), acc);
    y[part] = round_bf16(acc / (1.0f + expf(-acc)));
  }
  float sq = warp_sum(y[0] * y[0]), sk = warp_sum(y[1] * y[1]);
  if ((t & 31) == 0) {
    red[0][t >> 5] = sq;
    red[1][t >> 5] = sk;
  }
  if (t == 0) {
    const float av = a_raw + dt_bias_h;
    const float sp_ = av > 20.f ? av : log1pf(expf(av));
    gate_s[0] = 1.0f / (1.0f + expf(-b_raw));            // beta
    gate_s[1] = __expf(-expf(a_log_h) * sp_);            // exp(g)
  }
  __syncthreads();
  sq = (red[0][0] + red[0][1]) + (red[0][2] + red[0][3]);
  sk = (red[1][0] + red[1][1]) + (red[1][2] + red[1][3]);
  qf[t] = round_bf16(y[0] * rsqrtf(sq + 1e-6f) * 0.08838834764831845f);  // DK^-0.5
  kf[t] = round_bf16(y[1] * rsqrtf(sk + 1e-6f));
  __syncthreads();
  float o;
  gdn_token_update(s, kf, qf, gate_s[1], gate_s[0], y[2], o);
#pragma unroll
  for (int i = 0; i < GDN_D; ++i) __stcs(sp + i * GDN_D, s[i]);
  // gated RMSNorm over the head's 128 outputs
  const float x = round_bf16(o);
  const float ss = warp_sum(x * x);
  if ((t & 31) == 0) red[2][t >> 5] = ss;
  __syncthreads();
  const float rs = rsqrtf(((red[2][0] + red[2][1]) + (red[2][2] + red[2][3])) / static_cast<float>(GDN_D) + 1e-6f);
  out[(static_cast<int64_t>(b) * heads + h) * GDN_D + t] = __float2bfloat16_rn(x * rs * wv * (zv / (1.0f + expf(-zv))));
}

// ------------------------------------------------------------- streaming decode over column boxes (tensor-map TMA)
// The persistent pipeline with a finer grain and a copy warp of its own.  An item is a [128 rows x COLS columns] fp32 box
// of one head's state; ONE tensor-map TMA copy brings it into a ring of STAGES buffers and one takes it out.  A CTA is
// THREADS compute threads plus one copy warp: thread t of the compute part owns rows (t / COLS) * ROWS ... of column
// t % COLS, the row groups of a column meet through shared memory for k^T S and q^T S, and the copy warp alone waits
// for stores to drain before it reuses a buffer, so no compute thread ever stalls on a copy that is not its own item.
// Several such CTAs share an SM (their rings together hold most of its shared memory), which staggers the load,
// update and store phases that a single wave of register-resident heads runs in lockstep.  Needs the dense
// [B, H, 128, 128] state.
struct GdnRingParams {
  const __nv_bfloat16 *q, *k, *v;
  const float *beta, *g;
  __nv_bfloat16* out;
  int64_t q_b, q_h, k_b, k_h, v_b, v_h, be_b, be_h, g_b, g_h, o_b, o_h;
  int* err;
  int items, heads;  // items = batch * heads * (128 / COLS)
};

__device__ __forceinline__ void tma_load_2d(void* dst_smem, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst_smem)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, int c0, int c1, const void* src_smem) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(src_smem)), "r"(c0), "r"(c1)
               : "memory");
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

template <int COLS, int THREADS, int STAGES>
constexpr int gdn_ring_smem() { return STAGES * GDN_D * COLS * 4 + 128; }

template <int COLS, int THREADS, int STAGES, int CTAS>
__global__ void __launch_bounds__(THREADS + 32, CTAS)
gdn_decode_ring_kernel(const __grid_constant__ GdnRingParams p, const __grid_constant__ CUtensorMap map_state) {
  pdl_chain();
  constexpr int GROUPS = THREADS / COLS, ROWS = GDN_D / GROUPS, PER_HEAD = GDN_D / COLS, BOX = GDN_D * COLS;
  static_assert(THREADS >= GDN_D && THREADS % COLS == 0 && ROWS % 4 == 0, "ring kernel shape");
  extern __shared__ __align__(128) uint8_t ring_raw[];
  __shared__ uint64_t full[STAGES], done[STAGES];
  __shared__ __align__(16) float kf[GDN_D];
  __shared__ __align__(16) float qf[GDN_D];
  __shared__ float vf[COLS];
  __shared__ float red[2][GROUPS][COLS];  // [k^T S | q^T S][row group][column]
  __shared__ int failed;
  float* bufs = reinterpret_cast<float*>((reinterpret_cast<uintptr_t>(ring_raw) + 127) & ~uintptr_t(127));
  const int t = threadIdx.x;
  const int stride = static_cast<int>(gridDim.x), first = static_cast<int>(blockIdx.x);
  const int my_items = (p.items - first + stride - 1) / stride;
  if (t == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&done[s], THREADS);
    }
    failed = 0;
    mbar_fence_init();
    prefetch_tensormap(&map_state);
  }
  __syncthreads();

  if (t >= THREADS) {
    // ------------------------------------------------------------------------------------------- copy warp
    if (t != THREADS) return;
    auto load = [&](int n) {
      const int item = first + n * stride;
      mbar_expect_tx(&full[n % STAGES], BOX * 4);
      tma_load_2d(bufs + (n % STAGES) * BOX, &map_state, (item % PER_HEAD) * COLS, (item / PER_HEAD) * GDN_D,
                  &full[n % STAGES]);
    };
    const int ahead = min(my_items, STAGES);
    for (int n = 0; n < ahead; ++n) load(n);
    int loaded = ahead, n = 0;
    for (; n < my_items; ++n) {
      if (!mbar_wait_bounded(&done[n % STAGES], (n / STAGES) & 1)) break;  // the compute part gave up (or is lost)
      const int item = first + n * stride;
      tma_store_2d(&map_state, (item % PER_HEAD) * COLS, (item / PER_HEAD) * GDN_D, bufs + (n % STAGES) * BOX);
      if (n + STAGES < my_items) {
        bulk_wait_read();  // the store just issued has read its buffer: the box of item n + STAGES may land there
        load(n + STAGES);
        loaded = n + STAGES + 1;
      }
    }
    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");  // all stores complete before the CTA ends
    if (n < my_items) {
      atomicExch(p.err, 1);
      // boxes that were requested but never consumed may still be landing in this CTA's shared memory
      for (int m = n; m < loaded; ++m) mbar_wait_bounded(&full[m % STAGES], (m / STAGES) & 1, 1u << 12);
    }
    return;
  }

  // ------------------------------------------------------------------------------------------- compute part
  // Row group rg owns rows rg * ROWS + i; with boxes narrower than a warp two row groups share a warp and blocked rows
  // would put them on the same banks, so there the rows are dealt round-robin (row i * GROUPS + rg) and kf / qf are
  // stored in the matching order.
  constexpr bool DEALT = COLS < 32;
  const int c = t % COLS, rg = t / COLS;
  const int KSLOT = DEALT ? (t % GROUPS) * ROWS + t / GROUPS : t;
  // per-item operands of the NEXT item are fetched while the current one is computed
  float kn = 0.f, qn = 0.f, vn = 0.f, bn = 0.f, gn = 0.f;
  auto fetch = [&](int n) {
    const int item = first + n * stride, head = item / PER_HEAD, b = head / p.heads, h = head % p.heads;
    if (t < GDN_D) {
      kn = __bfloat162float(p.k[b * p.k_b + h * p.k_h + t]);
      qn = __bfloat162float(p.q[b * p.q_b + h * p.q_h + t]);
    }
    if (rg == 0) vn = __bfloat162float(p.v[b * p.v_b + h * p.v_h + (item % PER_HEAD) * COLS + c]);
    bn = p.beta[b * p.be_b + h * p.be_h];
    gn = p.g[b * p.g_b + h * p.g_h];
  };
  if (my_items > 0) fetch(0);
  for (int n = 0; n < my_items; ++n) {
    const int item = first + n * stride, head = item / PER_HEAD, b = head / p.heads, h = head % p.heads;
    float* buf = bufs + (n % STAGES) * BOX;
    const float eg = __expf(gn), bt = bn;
    // kf / qf / vf / red of the previous item are no longer read: every compute thread has passed that item's last
    // barrier, and the reads after it (red[1] for the output) are separated from the writes below by two more
    if (t < GDN_D) {
      kf[KSLOT] = kn;
      qf[KSLOT] = qn;
    }
    if (rg == 0) vf[c] = vn;
    if (n + 1 < my_items) fetch(n + 1);
    if (!mbar_wait_bounded(&full[n % STAGES], (n / STAGES) & 1)) failed = 1;
    named_barrier(1, THREADS);  // kf / qf / vf visible; the compute part agrees on whether the box arrived
    if (*reinterpret_cast<volatile int*>(&failed)) break;  // a lost copy: this item's state and output stay untouched
    float s[ROWS];
    float* col = DEALT ? buf + rg * COLS + c : buf + (rg * ROWS) * COLS + c;
    constexpr int RSTEP = DEALT ? GROUPS * COLS : COLS;  // floats between consecutive rows of this thread
    const float* kh = kf + rg * ROWS;
    const float* qh = qf + rg * ROWS;
    float m0 = 0.f, m1 = 0.f, m2 = 0.f, m3 = 0.f;
#pragma unroll
    for (int i = 0; i < ROWS; i += 4) {
      const float4 k4 = *reinterpret_cast<const float4*>(kh + i);
      s[i] = col[i * RSTEP] * eg;
      s[i + 1] = col[(i + 1) * RSTEP] * eg;
      s[i + 2] = col[(i + 2) * RSTEP] * eg;
      s[i + 3] = col[(i + 3) * RSTEP] * eg;
      m0 = fmaf(k4.x, s[i], m0);
      m1 = fmaf(k4.y, s[i + 1], m1);
      m2 = fmaf(k4.z, s[i + 2], m2);
      m3 = fmaf(k4.w, s[i + 3], m3);
    }
    red[0][rg][c] = (m0 + m1) + (m2 + m3);
    named_barrier(1, THREADS);
    float mem = 0.f;
#pragma unroll
    for (int r = 0; r < GROUPS; ++r) mem += red[0][r][c];
    const float delta = bt * (vf[c] - mem);
    float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
    for (int i = 0; i < ROWS; i += 4) {
      const float4 k4 = *reinterpret_cast<const float4*>(kh + i);
      const float4 q4 = *reinterpret_cast<const float4*>(qh + i);
      s[i] = fmaf(k4.x, delta, s[i]);
      s[i + 1] = fmaf(k4.y, delta, s[i + 1]);
      s[i + 2] = fmaf(k4.z, delta, s[i + 2]);
      s[i + 3] = fmaf(k4.w, delta, s[i + 3]);
      o0 = fmaf(q4.x, s[i], o0);
      o1 = fmaf(q4.y, s[i + 1], o1);
      o2 = fmaf(q4.z, s[i + 2], o2);
      o3 = fmaf(q4.w, s[i + 3], o3);
      col[i * RSTEP] = s[i];
      col[(i + 1) * RSTEP] = s[i + 1];
      col[(i + 2) * RSTEP] = s[i + 2];
      col[(i + 3) * RSTEP] = s[i + 3];
    }
    red[1][rg][c] = (o0 + o1) + (o2 + o3);
    fence_proxy_async();          // generic-proxy stores of the box before the TMA store reads them
    mbar_arrive(&done[n % STAGES]);  // the copy warp stores the box once all THREADS have arrived
    named_barrier(1, THREADS);
    if (rg == 0) {
      float o = 0.f;
#pragma unroll
      for (int r = 0; r < GROUPS; ++r) o += red[1][r][c];
      p.out[b * p.o_b + h * p.o_h + (item % PER_HEAD) * COLS + c] = __float2bfloat16_rn(o);
    }
  }
}

// fp32 map over the states seen as a matrix [batch * heads * 128 rows][128 columns]; a box is `cols` columns x 128 rows
static bool encode_state_map(CUtensorMap* map, const float* state, int64_t rows, int cols) {
  typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                               const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static std::atomic<EncodeFn> cached{nullptr};
  EncodeFn encode = cached.load();
  if (!encode) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess || fn == nullptr) {
      cudaGetLastError();
      return false;
    }
    encode = reinterpret_cast<EncodeFn>(fn);
    cached.store(encode);
  }
  const cuuint64_t dims[2] = {GDN_D, static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {GDN_D * 4};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(cols), GDN_D};
  const cuuint32_t es[2] = {1, 1};
  return encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(state), dims, strides, box, es,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Which form b200_gdn_recurrent_decode takes: 0 = chosen from the sizes; 1 one CTA per head, 2 one-warp slices, 3 ring of
// three [128 x 16] boxes, eight CTAs per SM (a form whose layout rules do not hold falls back to 1).
static std::atomic<int> g_gdn_decode_form{0};

template <int COLS, int THREADS, int STAGES, int CTAS>
static int launch_ring(GdnRingParams p, const float* state, int heads_total, cudaStream_t stream) {
  constexpr int SMEM = gdn_ring_smem<COLS, THREADS, STAGES>();
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    if (cudaFuncSetAttribute(gdn_decode_ring_kernel<COLS, THREADS, STAGES, CTAS>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess)
      return fail(ERR_RUNTIME, "gdn_recurrent_decode: cannot raise dynamic shared memory to %d", SMEM);
    configured[dev] = true;
  }
  CUtensorMap map;
  if (!encode_state_map(&map, state, static_cast<int64_t>(heads_total) * GDN_D, COLS))
    return fail(ERR_RUNTIME, "gdn_recurrent_decode: cannot encode the state tensor map");
  p.items = heads_total * (GDN_D / COLS);
  const int slots = CTAS * sm_count();
  const int grid = p.items < slots ? p.items : slots;
  launch_pdl(chain_overlap(), gdn_decode_ring_kernel<COLS, THREADS, STAGES, CTAS>, dim3(grid), dim3(THREADS + 32), SMEM, stream,
             p, map);
  return OK;
}

// ----------------------------------------------------------------- the whole mixer over the ring (large batches)
// gdn_decode_fused_kernel keeps a head's state in 128 registers per thread: two CTAs per SM, so 512 heads (B = 32) run
// as two waves that each load, compute and store in lockstep.  This form streams the state through the ring above
// instead: a CTA (128 compute threads + the copy warp) takes WHOLE heads - the head-wide steps (q/k norms, gated
// RMSNorm) stay inside it - as four [128 x 32] boxes each; four CTAs with three boxes in flight share an SM, every head
// of a 32-sequence batch is resident at once, and a head's conv / norm / gate chain runs while its first boxes are on
// their way.  A box is worked on as in gdn_decode_ring_kernel (thread = 32 rows of one column, the four row groups of a
// column meet in shared memory); the operands of the NEXT head of a CTA are fetched while the current head's boxes are
// worked on.  [128 x 16] boxes with six in flight (twice the barriers per head) measured 1.016 ms per whole-model step
// at B = 32 against 0.994 ms for this shape and 1.056 ms for the register form.
struct GdnMixerParams {
  const __nv_bfloat16* fused;  // read after pdl_wait(): no __restrict__ anywhere on this path
  int64_t fused_stride;
  __nv_bfloat16* conv_state;
  const __nv_bfloat16* w4;
  const float* a_log;
  const __nv_bfloat16* dt_bias;
  const float* norm_w;
  __nv_bfloat16* out;
  int* err;
  int heads_total, heads, overlap;
};

constexpr int MX_COLS = 32, MX_THREADS = GDN_D, MX_GROUPS = MX_THREADS / MX_COLS, MX_ROWS = GDN_D / MX_GROUPS;
constexpr int MX_PER_HEAD = GDN_D / MX_COLS, MX_BOX = GDN_D * MX_COLS;

template <int STAGES, int CTAS>
__global__ void __launch_bounds__(MX_THREADS + 32, CTAS)
gdn_mixer_ring_kernel(const __grid_constant__ GdnMixerParams p, const __grid_constant__ CUtensorMap map_state) {
  extern __shared__ __align__(128) uint8_t ring_raw[];
  __shared__ uint64_t full[STAGES], done[STAGES];
  __shared__ __align__(16) float kf[GDN_D];
  __shared__ __align__(16) float qf[GDN_D];
  __shared__ float vf[GDN_D];
  __shared__ float of[GDN_D];                      // the head's recurrence output, value column by value column
  __shared__ float red[2][MX_GROUPS][MX_COLS];     // [k^T S | q^T S][row group][column]
  __shared__ float nred[3][4];                     // per-warp sums of the three head-wide norms
  __shared__ float gate_s[2];
  __shared__ int failed;
  float* bufs = reinterpret_cast<float*>((reinterpret_cast<uintptr_t>(ring_raw) + 127) & ~uintptr_t(127));
  const int t = threadIdx.x;
  const int stride = static_cast<int>(gridDim.x), first = static_cast<int>(blockIdx.x);
  const int my_heads = (p.heads_total - first + stride - 1) / stride;
  const int my_items = my_heads * MX_PER_HEAD;
  const bool prefetch = (p.overlap & OVERLAP_PREFETCH) != 0;
  if (t == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&done[s], MX_THREADS);
    }
    failed = 0;
    mbar_fence_init();
    prefetch_tensormap(&map_state);
  }
  __syncthreads();
  if (p.overlap & OVERLAP_TRIGGER) pdl_trigger();
  // Without PREFETCH nothing is read before the kernel in front has finished.  With it the caller guarantees that the
  // conv state and the recurrent state were last written by an EARLIER kernel, so their loads go out first; `fused` is
  // read, and everything is stored, after the wait.
  if (!prefetch) pdl_wait();

  if (t >= MX_THREADS) {
    // ------------------------------------------------------------------------------------------- copy warp
    if (t != MX_THREADS) return;
    auto coords = [&](int n, int& x, int& y) {
      x = (n % MX_PER_HEAD) * MX_COLS;
      y = (first + (n / MX_PER_HEAD) * stride) * GDN_D;
    };
    auto load = [&](int n) {
      int x, y;
      coords(n, x, y);
      mbar_expect_tx(&full[n % STAGES], MX_BOX * 4);
      tma_load_2d(bufs + (n % STAGES) * MX_BOX, &map_state, x, y, &full[n % STAGES]);
    };
    const int ahead = min(my_items, STAGES);
    for (int n = 0; n < ahead; ++n) load(n);
    if (prefetch) pdl_wait();  // before the first store
    int loaded = ahead, n = 0;
    for (; n < my_items; ++n) {
      if (!mbar_wait_bounded(&done[n % STAGES], (n / STAGES) & 1)) break;  // the compute part gave up (or is lost)
      int x, y;
      coords(n, x, y);
      tma_store_2d(&map_state, x, y, bufs + (n % STAGES) * MX_BOX);
      if (n + STAGES < my_items) {
        bulk_wait_read();  // the store just issued has read its buffer: the box of item n + STAGES may land there
        load(n + STAGES);
        loaded = n + STAGES + 1;
      }
    }
    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");  // all stores complete before the CTA ends
    if (n < my_items) {
      atomicExch(p.err, 1);
      for (int m = n; m < loaded; ++m) mbar_wait_bounded(&full[m % STAGES], (m / STAGES) & 1, 1u << 12);
    }
    return;
  }

  // ------------------------------------------------------------------------------------------- compute part
  // thread t = channel t of the head's q, k, v and z slices in the head-wide steps; in a box it is column t % COLS of
  // row group t / COLS (boxes narrower than a warp: rows dealt round-robin, kf / qf stored in the matching order)
  const int c = t % MX_COLS, rg = t / MX_COLS;
  constexpr bool MX_DEALT = MX_COLS < 32;
  const int kslot = MX_DEALT ? (t % MX_GROUPS) * MX_ROWS + t / MX_GROUPS : t;
  const int kd = p.heads * GDN_D, width = 3 * kd;
  const float wv = p.norm_w[t];
  // operands of one head in registers: the three earlier conv rows, the four taps, then (after the wait) the new row
  __nv_bfloat16 cs[3][3], cw[3][4], cx[3], zraw, araw, braw;
  float a_log_h = 0.f, dt_bias_h = 0.f;
  auto fetch_state_side = [&](int head) {  // nothing the kernel in front writes
    const int b = head / p.heads, h = head % p.heads;
#pragma unroll
    for (int part = 0; part < 3; ++part) {
      const int ch = part * kd + h * GDN_D + t;
      const __nv_bfloat16* st = p.conv_state + static_cast<int64_t>(b) * 4 * width + ch;
      cs[part][0] = st[width];
      cs[part][1] = st[2 * width];
      cs[part][2] = st[3 * width];
#pragma unroll
      for (int r = 0; r < 4; ++r) cw[part][r] = p.w4[r * width + ch];
    }
    a_log_h = p.a_log[h];
    dt_bias_h = __bfloat162float(p.dt_bias[h]);
  };
  auto fetch_row_side = [&](int head) {  // the projection row: only after the wait
    const int b = head / p.heads, h = head % p.heads;
    const __nv_bfloat16* row = p.fused + static_cast<int64_t>(b) * p.fused_stride;
#pragma unroll
    for (int part = 0; part < 3; ++part) cx[part] = row[part * kd + h * GDN_D + t];
    zraw = row[width + h * GDN_D + t];
    araw = row[width + kd + h];
    braw = row[width + kd + p.heads + h];
  };
  if (my_heads > 0) fetch_state_side(first);
  if (prefetch) pdl_wait();
  if (my_heads > 0) fetch_row_side(first);

  for (int j = 0; j < my_heads; ++j) {
    const int head = first + j * stride, b = head / p.heads, h = head % p.heads;
    // ---- conv state shift + conv4 + SiLU, q/k L2 norms, gates (the fused kernel's arithmetic, rounding point by
    //      rounding point)
    float y[3];
#pragma unroll
    for (int part = 0; part < 3; ++part) {
      const int ch = part * kd + h * GDN_D + t;
      __nv_bfloat16* st = p.conv_state + static_cast<int64_t>(b) * 4 * width + ch;
      st[0] = cs[part][0];
      st[width] = cs[part][1];
      st[2 * width] = cs[part][2];
      st[3 * width] = cx[part];
      float acc = __bfloat162float(cw[part][0]) * __bfloat162float(cs[part][0]);
      acc = fmaf(__bfloat162float(cw[part][1]), __bfloat162float(cs[part][1]), acc);
      acc = fmaf(__bfloat162float(cw[part][2]), __bfloat162float(cs[part][2]), acc);
      acc = fmaf(__bfloat162float(cw[part][3]), __bfloat162float(cx[part]), acc);
      y[part] = round_bf16(acc / (1.0f + expf(-acc)));
    }
    const float zv = __bfloat162float(zraw);
    float sq = warp_sum(y[0] * y[0]), sk = warp_sum(y[1] * y[1]);
    if ((t & 31) == 0) {
      nred[0][t >> 5] = sq;
      nred[1][t >> 5] = sk;
    }
    if (t == 0) {
      const float av = __bfloat162float(araw) + dt_bias_h;
      const float sp_ = av > 20.f ? av : log1pf(expf(av));
      gate_s[0] = 1.0f / (1.0f + expf(-__bfloat162float(braw)));  // beta
      gate_s[1] = __expf(-expf(a_log_h) * sp_);                    // exp(g)
    }
    // the next head's operands start their way now and are used after this head's boxes
    if (j + 1 < my_heads) {
      fetch_state_side(head + stride);
      fetch_row_side(head + stride);
    }
    named_barrier(2, MX_THREADS);
    sq = (nred[0][0] + nred[0][1]) + (nred[0][2] + nred[0][3]);
    sk = (nred[1][0] + nred[1][1]) + (nred[1][2] + nred[1][3]);
    // kf / qf / vf of the previous head are no longer read: every compute thread has passed its last box's barriers
    qf[kslot] = round_bf16(y[0] * rsqrtf(sq + 1e-6f) * 0.08838834764831845f);  // DK^-0.5
    kf[kslot] = round_bf16(y[1] * rsqrtf(sk + 1e-6f));
    vf[t] = y[2];
    const float eg = gate_s[1], bt = gate_s[0];

    bool lost = false;
    for (int box = 0; box < MX_PER_HEAD; ++box) {
      const int n = j * MX_PER_HEAD + box;
      float* buf = bufs + (n % STAGES) * MX_BOX;
      if (!mbar_wait_bounded(&full[n % STAGES], (n / STAGES) & 1)) failed = 1;
      named_barrier(1, MX_THREADS);  // kf / qf / vf visible; the compute part agrees on whether the box arrived
      if (*reinterpret_cast<volatile int*>(&failed)) {
        lost = true;
        break;  // a lost copy: this box's state and the head's output stay untouched
      }
      float s[MX_ROWS];
      float* col = MX_DEALT ? buf + rg * MX_COLS + c : buf + (rg * MX_ROWS) * MX_COLS + c;
      constexpr int RSTEP = MX_DEALT ? MX_GROUPS * MX_COLS : MX_COLS;  // floats between consecutive rows of this thread
      const float* kh = kf + rg * MX_ROWS;
      const float* qh = qf + rg * MX_ROWS;
      float m0 = 0.f, m1 = 0.f, m2 = 0.f, m3 = 0.f;
#pragma unroll
      for (int i = 0; i < MX_ROWS; i += 4) {
        const float4 k4 = *reinterpret_cast<const float4*>(kh + i);
        s[i] = col[i * RSTEP] * eg;
        s[i + 1] = col[(i + 1) * RSTEP] * eg;
        s[i + 2] = col[(i + 2) * RSTEP] * eg;
        s[i + 3] = col[(i + 3) * RSTEP] * eg;
        m0 = fmaf(k4.x, s[i], m0);
        m1 = fmaf(k4.y, s[i + 1], m1);
        m2 = fmaf(k4.z, s[i + 2], m2);
        m3 = fmaf(k4.w, s[i + 3], m3);
      }
      red[0][rg][c] = (m0 + m1) + (m2 + m3);
      named_barrier(1, MX_THREADS);
      float mem = 0.f;
#pragma unroll
      for (int r = 0; r < MX_GROUPS; ++r) mem += red[0][r][c];
      const float delta = bt * (vf[box * MX_COLS + c] - mem);
      float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
      for (int i = 0; i < MX_ROWS; i += 4) {
        const float4 k4 = *reinterpret_cast<const float4*>(kh + i);
        const float4 q4 = *reinterpret_cast<const float4*>(qh + i);
        s[i] = fmaf(k4.x, delta, s[i]);
        s[i + 1] = fmaf(k4.y, delta, s[i + 1]);
        s[i + 2] = fmaf(k4.z, delta, s[i + 2]);
        s[i + 3] = fmaf(k4.w, delta, s[i + 3]);
        o0 = fmaf(q4.x, s[i], o0);
        o1 = fmaf(q4.y, s[i + 1], o1);
        o2 = fmaf(q4.z, s[i + 2], o2);
        o3 = fmaf(q4.w, s[i + 3], o3);
        col[i * RSTEP] = s[i];
        col[(i + 1) * RSTEP] = s[i + 1];
        col[(i + 2) * RSTEP] = s[i + 2];
        col[(i + 3) * RSTEP] = s[i + 3];
      }
      red[1][rg][c] = (o0 + o1) + (o2 + o3);
      fence_proxy_async();             // generic-proxy stores of the box before the TMA store reads them
      mbar_arrive(&done[n % STAGES]);  // the copy warp stores the box once all compute threads have arrived
      named_barrier(1, MX_THREADS);
      if (rg == 0) {
        float o = 0.f;
#pragma unroll
        for (int r = 0; r < MX_GROUPS; ++r) o += red[1][r][c];
        of[box * MX_COLS + c] = o;
      }
    }
    if (lost) break;
    // ---- gated RMSNorm over the head's 128 outputs
    named_barrier(2, MX_THREADS);  // `of` complete
    const float x = round_bf16(of[t]);
    const float ss = warp_sum(x * x);
    if ((t & 31) == 0) nred[2][t >> 5] = ss;
    named_barrier(2, MX_THREADS);
    const float rs = rsqrtf(((nred[2][0] + nred[2][1]) + (nred[2][2] + nred[2][3])) / static_cast<float>(GDN_D) + 1e-6f);
    p.out[(static_cast<int64_t>(b) * p.heads + h) * GDN_D + t] = __float2bfloat16_rn(x * rs * wv * (zv / (1.0f + expf(-zv))));
  }
}

constexpr int MX_STAGES = 3, MX_CTAS = 4;

constexpr int SEQ_TILE = 16;  // tokens staged in shared memory per step of the prefill loop

__global__ void __launch_bounds__(GDN_THREADS)
gdn_sequential_kernel(const __nv_bfloat16* __restrict__ q, int64_t q_t, int64_t q_h,
                      const __nv_bfloat16* __restrict__ k, int64_t k_t, int64_t k_h,
                      const __nv_bfloat16* __restrict__ v, int64_t v_t, int64_t v_h, const float* __restrict__ beta,
                      int64_t be_t, int64_t be_h, const float* __restrict__ g, int64_t g_t, int64_t g_h,
                      const int32_t* __restrict__ cu_seqlens, int total_tokens, float* __restrict__ state,
                      __nv_bfloat16* __restrict__ out, int64_t o_t, int64_t o_h, int heads) {
  __shared__ __align__(16) float kf[SEQ_TILE][GDN_D];
  __shared__ __align__(16) float qf[SEQ_TILE][GDN_D];
  __shared__ float vf[SEQ_TILE][GDN_D];
  __shared__ float egf[SEQ_TILE], btf[SEQ_TILE];
  const int b = blockIdx.x / heads, h = blockIdx.x % heads, col = threadIdx.x;
  const int seq_start = cu_seqlens ? cu_seqlens[b] : 0;
  const int seq_len = (cu_seqlens ? cu_seqlens[b + 1] : total_tokens) - seq_start;
  float s[GDN_D];
#pragma unroll
  for (int i = 0; i < GDN_D; ++i) s[i] = 0.f;

  for (int t0 = 0; t0 < seq_len; t0 += SEQ_TILE) {
    const int nt = min(SEQ_TILE, seq_len - t0);
    __syncthreads();  // previous tile fully consumed
    for (int j = 0; j < nt; ++j) {
      const int64_t t = seq_start + t0 + j;
      kf[j][col] = __bfloat162float(k[t * k_t + h * k_h + col]);
      qf[j][col] = __bfloat162float(q[t * q_t + h * q_h + col]);
      vf[j][col] = __bfloat162float(v[t * v_t + h * v_h + col]);
    }
    if (col < nt) {
      const int64_t t = seq_start + t0 + col;
      egf[col] = __expf(g[t * g_t + h * g_h]);
      btf[col] = beta[t * be_t + h * be_h];
    }
    __syncthreads();
    for (int j = 0; j < nt; ++j) {
      float o;
      gdn_token_update(s, kf[j], qf[j], egf[j], btf[j], vf[j][col], o);
      out[(seq_start + t0 + j) * o_t + h * o_h + col] = __float2bfloat16_rn(o);
    }
  }
  float* sp = state + (static_cast<int64_t>(b) * heads + h) * GDN_D * GDN_D + col;
#pragma unroll
  for (int i = 0; i < GDN_D; ++i) sp[i * GDN_D] = s[i];
}

}  // namespace b200

using namespace b200;

extern "C" int b200_gdn_recurrent_decode(const void* q, int64_t q_stride_b, int64_t q_stride_h, const void* k,
                                         int64_t k_stride_b, int64_t k_stride_h, const void* v, int64_t v_stride_b,
                                         int64_t v_stride_h, const float* beta, int64_t beta_stride_b,
                                         int64_t beta_stride_h, const float* g, int64_t g_stride_b, int64_t g_stride_h,
                                         float* state, int64_t state_stride_b, int64_t state_stride_h, void* out,
                                         int64_t out_stride_b, int64_t out_stride_h, int32_t batch, int32_t num_heads,
                                         int32_t key_dim, int32_t value_dim, b200_stream_t stream) {
  B200_REQUIRE(batch > 0 && num_heads > 0, "gdn_recurrent_decode: empty shape");
  B200_REQUIRE(key_dim == GDN_D && value_dim == GDN_D, "gdn_recurrent_decode: key/value dim must be %d (got %d/%d)",
               GDN_D, key_dim, value_dim);
  const bool dense = (reinterpret_cast<uintptr_t>(state) % 128 == 0) && state_stride_h == GDN_D * GDN_D &&
                     state_stride_b == static_cast<int64_t>(num_heads) * GDN_D * GDN_D;
  const bool slices_ok = (reinterpret_cast<uintptr_t>(q) % 8 == 0) && (reinterpret_cast<uintptr_t>(k) % 8 == 0) &&
                         q_stride_b % 4 == 0 && q_stride_h % 4 == 0 && k_stride_b % 4 == 0 && k_stride_h % 4 == 0;
  const int items = batch * num_heads;
  int form = g_gdn_decode_form.load();
  if (form == 0) {
    // Measured on B200 (16 heads per sequence, batch 1 ... 256): the ring wins or ties up to sixteen heads per SM
    // (batch 128), the one-warp slices beyond (batch 256: 0.99 of the copy bandwidth against 0.87).
    form = (dense && items <= 16 * sm_count()) ? 3 : (slices_ok ? 2 : 1);
  }
  if ((form >= 3 && !dense) || (form == 2 && !slices_ok)) form = 1;
  if (form >= 3) {
    GdnRingParams p;
    p.q = static_cast<const __nv_bfloat16*>(q);
    p.k = static_cast<const __nv_bfloat16*>(k);
    p.v = static_cast<const __nv_bfloat16*>(v);
    p.beta = beta;
    p.g = g;
    p.out = static_cast<__nv_bfloat16*>(out);
    p.q_b = q_stride_b; p.q_h = q_stride_h; p.k_b = k_stride_b; p.k_h = k_stride_h; p.v_b = v_stride_b; p.v_h = v_stride_h;
    p.be_b = beta_stride_b; p.be_h = beta_stride_h; p.g_b = g_stride_b; p.g_h = g_stride_h;
    p.o_b = out_stride_b; p.o_h = out_stride_h;
    p.err = wait_timeout_flag();
    if (!p.err) return fail(ERR_RUNTIME, "gdn_recurrent_decode: no error flag");
    p.heads = num_heads;
    const cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const int rc = launch_ring<16, 128, 3, 8>(p, state, items, st);
    if (rc != OK) return rc;
    return check_launch("gdn_recurrent_decode");
  }
  // the one-warp slices keep the SMs evenly loaded and shorten the last wave; q and k rows must allow 8-byte loads
  if (form == 2) {
    launch_pdl(chain_overlap(), gdn_decode_slice_kernel, dim3(static_cast<unsigned>(items) * (GDN_D / GDN_SLICE)), dim3(GDN_SLICE), 0, reinterpret_cast<cudaStream_t>(stream),
             
        static_cast<const __nv_bfloat16*>(q), q_stride_b, q_stride_h, static_cast<const __nv_bfloat16*>(k), k_stride_b,
        k_stride_h, static_cast<const __nv_bfloat16*>(v), v_stride_b, v_stride_h, beta, beta_stride_b, beta_stride_h, g,
        g_stride_b, g_stride_h, state, state_stride_b, state_stride_h, static_cast<__nv_bfloat16*>(out), out_stride_b,
        out_stride_h, num_heads);
    return check_launch("gdn_recurrent_decode");
  }
  launch_pdl(chain_overlap(), gdn_decode_kernel, dim3(static_cast<unsigned>(batch) * num_heads), dim3(GDN_THREADS), 0, reinterpret_cast<cudaStream_t>(stream),
             
      static_cast<const __nv_bfloat16*>(q), q_stride_b, q_stride_h, static_cast<const __nv_bfloat16*>(k), k_stride_b,
      k_stride_h, static_cast<const __nv_bfloat16*>(v), v_stride_b, v_stride_h, beta, beta_stride_b, beta_stride_h, g,
      g_stride_b, g_stride_h, state, state_stride_b, state_stride_h, static_cast<__nv_bfloat16*>(out), out_stride_b,
      out_stride_h, num_heads);
  return check_launch("gdn_recurrent_decode");
}

extern "C" int b200_gdn_recurrent_decode_form(int32_t form) {
  B200_REQUIRE(form >= 0 && form <= 3, "gdn_recurrent_decode_form: form must be 0..3 (got %d)", form);
  g_gdn_decode_form.store(form);
  return OK;
}

extern "C" int b200_gdn_decode_fused(const void* fused, int64_t fused_stride, void* conv_state, const void* weight4,
                                     const float* a_log, const void* dt_bias, const float* norm_weight, float* state,
                                     void* out, int32_t batch, int32_t num_heads, int32_t head_dim,
                                     int32_t overlap, b200_stream_t stream) {
  B200_REQUIRE(batch > 0 && num_heads > 0 && head_dim == GDN_D, "gdn_decode_fused: head_dim must be %d (got %d)", GDN_D,
               head_dim);
  // More heads than two register-resident CTAs per SM can hold at once: the ring form (b200_gdn_recurrent_decode_form
  // 1 / 3 force either form here too).
  const int64_t heads_total = static_cast<int64_t>(batch) * num_heads;
  const int form = g_gdn_decode_form.load();
  const bool ring_ok = aligned16(state) && heads_total * GDN_D < (1LL << 31);
  if (ring_ok && (form == 3 || (form != 1 && heads_total > 2 * sm_count()))) {
    constexpr int SMEM = MX_STAGES * MX_BOX * 4 + 128;
    static bool configured[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
      if (cudaFuncSetAttribute(gdn_mixer_ring_kernel<MX_STAGES, MX_CTAS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               SMEM) != cudaSuccess)
        return fail(ERR_RUNTIME, "gdn_decode_fused: cannot raise dynamic shared memory to %d", SMEM);
      configured[dev] = true;
    }
    CUtensorMap map;
    if (!encode_state_map(&map, state, heads_total * GDN_D, MX_COLS))
      return fail(ERR_RUNTIME, "gdn_decode_fused: cannot encode the state tensor map");
    GdnMixerParams p;
    p.fused = static_cast<const __nv_bfloat16*>(fused);
    p.fused_stride = fused_stride;
    p.conv_state = static_cast<__nv_bfloat16*>(conv_state);
    p.w4 = static_cast<const __nv_bfloat16*>(weight4);
    p.a_log = a_log;
    p.dt_bias = static_cast<const __nv_bfloat16*>(dt_bias);
    p.norm_w = norm_weight;
    p.out = static_cast<__nv_bfloat16*>(out);
    p.err = wait_timeout_flag();
    if (!p.err) return fail(ERR_RUNTIME, "gdn_decode_fused: no error flag");
    p.heads_total = static_cast<int>(heads_total);
    p.heads = num_heads;
    p.overlap = overlap;
    const int slots = MX_CTAS * sm_count();
    const int grid = heads_total < slots ? static_cast<int>(heads_total) : slots;
    if (launch_pdl((overlap & OVERLAP_START) != 0, gdn_mixer_ring_kernel<MX_STAGES, MX_CTAS>, dim3(grid),
                   dim3(MX_THREADS + 32), SMEM, reinterpret_cast<cudaStream_t>(stream), p, map) != cudaSuccess)
      return fail(ERR_LAUNCH, "gdn_decode_fused: %s", cudaGetErrorString(cudaGetLastError()));
    return check_launch("gdn_decode_fused");
  }
  if (launch_pdl((overlap & OVERLAP_START) != 0, gdn_decode_fused_kernel, dim3(static_cast<unsigned>(batch) * num_heads), dim3(GDN_THREADS), 0,
                 reinterpret_cast<cudaStream_t>(stream), static_cast<const __nv_bfloat16*>(fused), fused_stride,
                 static_cast<__nv_bfloat16*>(conv_state), static_cast<const __nv_bfloat16*>(weight4), a_log,
                 static_cast<const __nv_bfloat16*>(dt_bias), norm_weight, state, static_cast<__nv_bfloat16*>(out),
                 num_heads, overlap) != cudaSuccess)
    return fail(ERR_LAUNCH, "gdn_decode_fused: %s", cudaGetErrorString(cudaGetLastError()));
  return check_launch("gdn_decode_fused");
}

extern "C" int b200_gdn_recurrent_prefill_sequential(
    const void* q, int64_t q_stride_t, int64_t q_stride_h, const void* k, int64_t k_stride_t, int64_t k_stride_h,
    const void* v, int64_t v_stride_t, int64_t v_stride_h, const float* beta, int64_t beta_stride_t,
    int64_t beta_stride_h, const float* g, int64_t g_stride_t, int64_t g_stride_h, const int32_t* cu_seqlens,
    int32_t batch, int32_t total_tokens, float* state, void* out, int64_t out_stride_t, int64_t out_stride_h,
    int32_t num_heads, int32_t key_dim, int32_t value_dim, b200_stream_t stream) {
  B200_REQUIRE(batch > 0 && num_heads > 0 && total_tokens > 0, "gdn_recurrent_prefill_sequential: empty shape");
  B200_REQUIRE(key_dim == GDN_D && value_dim == GDN_D,
               "gdn_recurrent_prefill_sequential: key/value dim must be %d (got %d/%d)", GDN_D, key_dim, value_dim);
  B200_REQUIRE(cu_seqlens != nullptr || batch == 1, "gdn_recurrent_prefill_sequential: batch > 1 needs cu_seqlens");
  gdn_sequential_kernel<<<static_cast<unsigned>(batch) * num_heads, GDN_THREADS, 0,
                          reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(q), q_stride_t, q_stride_h, static_cast<const __nv_bfloat16*>(k), k_stride_t,
      k_stride_h, static_cast<const __nv_bfloat16*>(v), v_stride_t, v_stride_h, beta, beta_stride_t, beta_stride_h, g,
      g_stride_t, g_stride_h, cu_seqlens, total_tokens, state, static_cast<__nv_bfloat16*>(out), out_stride_t,
      out_stride_h, num_heads);
  return check_launch("gdn_recurrent_prefill_sequential");
}
