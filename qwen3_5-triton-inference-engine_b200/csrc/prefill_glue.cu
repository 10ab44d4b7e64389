// Element-wise operators of the Gated-DeltaNet input pipeline and of the residual stream, each one launch, for prompts
// (many tokens) as well as for decode batches:
//   b200_conv4_prefill                   <-> triton_kernels/depthwise_causal_conv4_prefill.py:18-91 (op :108-170)
//   b200_conv4_decode                    <-> triton_kernels/depthwise_causal_conv4_decode.py:78-149 (op :152-207)
//   b200_conv_state_from_packed_prefill  <-> triton_kernels/depthwise_causal_conv4_decode.py:254-329 (op :332-374)
//   b200_gdn_qk_norm_gates               <-> triton_kernels/gdn_qk_norm_gates.py:14-114 (op :128-200)
//   b200_embedding_gather                <-> triton_kernels/embedding_gather.py:14-49
//   b200_residual_add                    <-> triton_kernels/residual_add.py:7-20
// All are HBM bound: a thread moves 16 bytes (8 bf16 channels) per access, the math is fp32 with one rounding to bf16
// where the reference rounds.
#include "b200_attn.h"
#include "common.cuh"

namespace b200 {

__device__ __forceinline__ void unpack8g(const uint4& v, float (&f)[8]) {
  f[0] = bf16_lo(v.x); f[1] = bf16_hi(v.x); f[2] = bf16_lo(v.y); f[3] = bf16_hi(v.y);
  f[4] = bf16_lo(v.z); f[5] = bf16_hi(v.z); f[6] = bf16_lo(v.w); f[7] = bf16_hi(v.w);
}
__device__ __forceinline__ uint4 pack8g(const float (&f)[8]) {
  return make_uint4(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]), pack_bf16(f[4], f[5]), pack_bf16(f[6], f[7]));
}
// acc * sigmoid(acc).  exp through ex2.approx and the division through rcp.approx (2 ulp each - what the reference's
// Triton kernel itself compiles to on a GPU): the result is rounded to bf16 (8 bits), which these 22-bit-accurate steps
// move for about one element in a thousand, by one bf16 ulp.
__device__ __forceinline__ float silu_ref(float a) { return silu_fast(a); }

// ---------------------------------------------------------------------------------------- depthwise conv4 + SiLU
// y[t,c] = silu(sum_r w[c,r] * x[t+r-3, c]); a tap whose row lies before seq_start[t] (the first row of t's own
// sequence in the packed buffer) reads zero.  One thread = 8 channels of CONV_TPT consecutive tokens: it issues its
// CONV_TPT + 3 row loads and its weight loads before the first use and keeps no loop-carried window, so a thread costs
// 11 16-byte loads per 4 outputs, the 32 taps are unpacked once per 4 tokens, and ~20 warps per SM stay resident.  A
// warp is 4 tokens x 256 channels (512 contiguous bytes per row), a CTA 16 consecutive tokens, whose warps find each
// other's rows in the L1.  Only a thread whose four tokens belong to two sequences takes the masked path.
constexpr int CONV_THREADS = 128;
constexpr int CONV_TPT = 4;                               // tokens per thread (prefill kernel)
constexpr int CONV_TOKENS = CONV_THREADS / 32 * CONV_TPT;  // tokens per CTA (prefill kernel)

__global__ void __launch_bounds__(CONV_THREADS)
conv4_prefill_kernel(const __nv_bfloat16* __restrict__ x, int64_t x_stride_t, const __nv_bfloat16* __restrict__ w,
                     int64_t w_stride_d, int64_t w_stride_k, const int32_t* __restrict__ seq_start,
                     __nv_bfloat16* __restrict__ out, int64_t out_stride_t, int tokens, int channels) {
  const int t0 = (blockIdx.x * (CONV_THREADS / 32) + (threadIdx.x >> 5)) * CONV_TPT;
  const int c = (blockIdx.y * 32 + (threadIdx.x & 31)) * 8;
  if (t0 >= tokens || c >= channels) return;
  int lower[CONV_TPT];
  int lowest = tokens, highest = 0;
#pragma unroll
  for (int j = 0; j < CONV_TPT; ++j) {
    lower[j] = seq_start != nullptr ? max(seq_start[min(t0 + j, tokens - 1)], 0) : 0;
    lowest = min(lowest, lower[j]);
    highest = max(highest, lower[j]);
  }
  uint4 rows[CONV_TPT + 3];
#pragma unroll
  for (int r = 0; r < CONV_TPT + 3; ++r) {
    const int tr = t0 - 3 + r;
    rows[r] = (tr >= lowest && tr < tokens) ? *reinterpret_cast<const uint4*>(x + static_cast<int64_t>(tr) * x_stride_t + c)
                                            : make_uint4(0, 0, 0, 0);
  }
  float wt[4][8];
  if (w_stride_k == 1 && w_stride_d == 4 && (reinterpret_cast<uintptr_t>(w) & 15) == 0) {
    // [channels, 4] contiguous: the 32 taps of this thread are 64 consecutive bytes
    const uint4* wp = reinterpret_cast<const uint4*>(w + static_cast<int64_t>(c) * 4);
#pragma unroll
    for (int q = 0; q < 4; ++q) {  // two channels per 16 bytes
      const uint4 v = wp[q];
      const uint32_t u[4] = {v.x, v.y, v.z, v.w};
      wt[0][2 * q] = bf16_lo(u[0]);
      wt[1][2 * q] = bf16_hi(u[0]);
      wt[2][2 * q] = bf16_lo(u[1]);
      wt[3][2 * q] = bf16_hi(u[1]);
      wt[0][2 * q + 1] = bf16_lo(u[2]);
      wt[1][2 * q + 1] = bf16_hi(u[2]);
      wt[2][2 * q + 1] = bf16_lo(u[3]);
      wt[3][2 * q + 1] = bf16_hi(u[3]);
    }
  } else {
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
      for (int j = 0; j < 8; ++j) wt[r][j] = __bfloat162float(w[(c + j) * w_stride_d + r * w_stride_k]);
  }
  float xr[CONV_TPT + 3][8];
#pragma unroll
  for (int r = 0; r < CONV_TPT + 3; ++r) unpack8g(rows[r], xr[r]);
  // rows below `lowest` were zeroed as they were loaded, which is the whole mask when all of this thread's tokens belong
  // to one sequence
  const bool inside = highest == lowest;
#pragma unroll
  for (int j = 0; j < CONV_TPT; ++j) {
    const int t = t0 + j;
    if (t >= tokens) break;
    float o[8];
    if (inside) {
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        // the reference sums the four products in tap order (its compiled kernel contracts them into fused multiply-adds)
        float acc = xr[j][e] * wt[0][e];
        acc = fmaf(xr[j + 1][e], wt[1][e], acc);
        acc = fmaf(xr[j + 2][e], wt[2][e], acc);
        acc = fmaf(xr[j + 3][e], wt[3][e], acc);
        o[e] = silu_ref(acc);
      }
    } else {
      const int first = lower[j] - (t - 3);  // taps below `first` lie before the token's own sequence
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        float acc = (first <= 0 ? xr[j][e] : 0.f) * wt[0][e];
        acc = fmaf(first <= 1 ? xr[j + 1][e] : 0.f, wt[1][e], acc);
        acc = fmaf(first <= 2 ? xr[j + 2][e] : 0.f, wt[2][e], acc);
        acc = fmaf(first <= 3 ? xr[j + 3][e] : 0.f, wt[3][e], acc);
        o[e] = silu_ref(acc);
      }
    }
    *reinterpret_cast<uint4*>(out + static_cast<int64_t>(t) * out_stride_t + c) = pack8g(o);
  }
}

// One token per sequence: state[b] (the last 4 conv INPUT rows) shifts up by one row, x[b] becomes row 3, then the same
// sum over the 4 rows.  grid = (sequence, 1024-channel block).
__global__ void __launch_bounds__(CONV_THREADS)
conv4_decode_kernel(const __nv_bfloat16* x, int64_t x_stride_b, __nv_bfloat16* state,
                    const __nv_bfloat16* w4, __nv_bfloat16* out, int64_t out_stride_b,
                    int channels) {
  pdl_chain();
  const int c = (blockIdx.y * CONV_THREADS + threadIdx.x) * 8;
  if (c >= channels) return;
  const int b = blockIdx.x;
  __nv_bfloat16* st = state + static_cast<int64_t>(b) * 4 * channels + c;
  const uint4 r1 = *reinterpret_cast<const uint4*>(st + channels);
  const uint4 r2 = *reinterpret_cast<const uint4*>(st + 2 * channels);
  const uint4 r3 = *reinterpret_cast<const uint4*>(st + 3 * channels);
  const uint4 xn = *reinterpret_cast<const uint4*>(x + b * x_stride_b + c);
  *reinterpret_cast<uint4*>(st) = r1;
  *reinterpret_cast<uint4*>(st + channels) = r2;
  *reinterpret_cast<uint4*>(st + 2 * channels) = r3;
  *reinterpret_cast<uint4*>(st + 3 * channels) = xn;
  float row[4][8], wt[4][8], o[8];
  unpack8g(r1, row[0]);
  unpack8g(r2, row[1]);
  unpack8g(r3, row[2]);
  unpack8g(xn, row[3]);
#pragma unroll
  for (int r = 0; r < 4; ++r) unpack8g(*reinterpret_cast<const uint4*>(w4 + r * channels + c), wt[r]);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    float acc = __fmul_rn(row[0][j], wt[0][j]);
    acc = __fadd_rn(acc, __fmul_rn(row[1][j], wt[1][j]));
    acc = __fadd_rn(acc, __fmul_rn(row[2][j], wt[2][j]));
    acc = __fadd_rn(acc, __fmul_rn(row[3][j], wt[3][j]));
    o[j] = silu_ref(acc);
  }
  *reinterpret_cast<uint4*>(out + b * out_stride_b + c) = pack8g(o);
}

// state[b, r, :] = x[end_b - 4 + r, :] when that row belongs to sequence b, else zero.
__global__ void __launch_bounds__(CONV_THREADS)
conv_state_pack_kernel(__nv_bfloat16* __restrict__ state, const __nv_bfloat16* __restrict__ x, int64_t x_stride_t,
                       const int32_t* __restrict__ cu_seqlens, int channels) {
  const int c = (blockIdx.y * CONV_THREADS + threadIdx.x) * 8;
  if (c >= channels) return;
  const int b = blockIdx.x;
  const int start = cu_seqlens[b], end = cu_seqlens[b + 1];
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int t = end - 4 + r;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (t >= start) v = *reinterpret_cast<const uint4*>(x + static_cast<int64_t>(t) * x_stride_t + c);
    *reinterpret_cast<uint4*>(state + (static_cast<int64_t>(b) * 4 + r) * channels + c) = v;
  }
}

// ------------------------------------------------------------------------------- q/k L2 norms, beta and g gates
// One warp per (token, head) row of 128: q_n = q * rsqrt(sum q^2 + 1e-6) * 128^-0.5, k_n = k * rsqrt(sum k^2 + 1e-6),
// both rounded to bf16; beta = sigmoid(b), g = -exp(a_log) * softplus(a + dt_bias) in fp32.
__global__ void __launch_bounds__(128)
gdn_qk_norm_gates_kernel(const __nv_bfloat16* q, int64_t q_t, int64_t q_h,
                         const __nv_bfloat16* k, int64_t k_t, int64_t k_h,
                         const __nv_bfloat16* a, int64_t a_t, const __nv_bfloat16* b,
                         int64_t b_t, const float* a_log, const __nv_bfloat16* dt_bias,
                         __nv_bfloat16* q_out, __nv_bfloat16* k_out, float* beta,
                         float* g, int64_t rows, int heads) {
  pdl_chain();
  const int64_t row = static_cast<int64_t>(blockIdx.x) * 4 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const int64_t t = row / heads;
  const int h = static_cast<int>(row % heads);
  const uint2 qv = *reinterpret_cast<const uint2*>(q + t * q_t + h * q_h + lane * 4);
  const uint2 kv = *reinterpret_cast<const uint2*>(k + t * k_t + h * k_h + lane * 4);
  const float qf[4] = {bf16_lo(qv.x), bf16_hi(qv.x), bf16_lo(qv.y), bf16_hi(qv.y)};
  const float kf[4] = {bf16_lo(kv.x), bf16_hi(kv.x), bf16_lo(kv.y), bf16_hi(kv.y)};
  const float sq = warp_sum((qf[0] * qf[0] + qf[1] * qf[1]) + (qf[2] * qf[2] + qf[3] * qf[3]));
  const float sk = warp_sum((kf[0] * kf[0] + kf[1] * kf[1]) + (kf[2] * kf[2] + kf[3] * kf[3]));
  const float rq = rsqrtf(sq + 1e-6f), rk = rsqrtf(sk + 1e-6f);
  constexpr float Q_SCALE = 0.08838834764831845f;  // 128^-0.5
  float qo[4], ko[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    qo[j] = __fmul_rn(__fmul_rn(qf[j], rq), Q_SCALE);
    ko[j] = __fmul_rn(kf[j], rk);
  }
  *reinterpret_cast<uint2*>(q_out + row * GDN_D + lane * 4) = make_uint2(pack_bf16(qo[0], qo[1]), pack_bf16(qo[2], qo[3]));
  *reinterpret_cast<uint2*>(k_out + row * GDN_D + lane * 4) = make_uint2(pack_bf16(ko[0], ko[1]), pack_bf16(ko[2], ko[3]));
  if (lane == 0) {
    const float bv = __bfloat162float(b[t * b_t + h]);
    const float sp_in = __bfloat162float(a[t * a_t + h]) + __bfloat162float(dt_bias[h]);
    const float sp = fmaxf(sp_in, 0.f) + logf(1.0f + expf(-fabsf(sp_in)));
    beta[row] = 1.0f / (1.0f + expf(-bv));
    g[row] = -expf(a_log[h]) * sp;
  }
}

// The same for prompt-sized inputs (16-byte aligned rows): 16 lanes x 8 elements per row, eight rows per CTA, so each
// thread has two 16-byte loads in flight; the gates of the CTA's eight rows are computed by its first eight threads,
// whose a / b loads are issued with the row loads.
__global__ void __launch_bounds__(128)
gdn_qk_norm_gates_wide_kernel(const __nv_bfloat16* q, int64_t q_t, int64_t q_h,
                              const __nv_bfloat16* k, int64_t k_t, int64_t k_h,
                              const __nv_bfloat16* a, int64_t a_t, const __nv_bfloat16* b,
                              int64_t b_t, const float* a_log, const __nv_bfloat16* dt_bias,
                              __nv_bfloat16* q_out, __nv_bfloat16* k_out, float* beta,
                              float* g, int64_t rows, int heads) {
  pdl_chain();
  const int sub = threadIdx.x & 15;
  const int64_t row_raw = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 4);
  const bool live = row_raw < rows;
  const int64_t row = live ? row_raw : rows - 1;  // a dead half-warp repeats the last row and stores nothing
  const int64_t t = row / heads;
  const int h = static_cast<int>(row % heads);
  const uint4 qv = *reinterpret_cast<const uint4*>(q + t * q_t + h * q_h + sub * 8);
  const uint4 kv = *reinterpret_cast<const uint4*>(k + t * k_t + h * k_h + sub * 8);
  const int64_t gate_row = static_cast<int64_t>(blockIdx.x) * 8 + threadIdx.x;
  const bool gate_thread = threadIdx.x < 8 && gate_row < rows;
  float bv = 0.f, sp_in = 0.f, decay = 0.f;
  if (gate_thread) {
    const int64_t gt = gate_row / heads;
    const int gh = static_cast<int>(gate_row % heads);
    bv = __bfloat162float(b[gt * b_t + gh]);
    sp_in = __bfloat162float(a[gt * a_t + gh]) + __bfloat162float(dt_bias[gh]);
    decay = a_log[gh];
  }
  float qf[8], kf[8];
  unpack8g(qv, qf);
  unpack8g(kv, kf);
  float sq = 0.f, sk = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    sq = fmaf(qf[j], qf[j], sq);
    sk = fmaf(kf[j], kf[j], sk);
  }
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) {
    sq += __shfl_xor_sync(0xffffffffu, sq, o);
    sk += __shfl_xor_sync(0xffffffffu, sk, o);
  }
  const float rq = rsqrtf(sq + 1e-6f), rk = rsqrtf(sk + 1e-6f);
  constexpr float Q_SCALE = 0.08838834764831845f;  // 128^-0.5
  float qo[8], ko[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    qo[j] = __fmul_rn(__fmul_rn(qf[j], rq), Q_SCALE);
    ko[j] = __fmul_rn(kf[j], rk);
  }
  if (live) {
    *reinterpret_cast<uint4*>(q_out + row * GDN_D + sub * 8) = pack8g(qo);
    *reinterpret_cast<uint4*>(k_out + row * GDN_D + sub * 8) = pack8g(ko);
  }
  if (gate_thread) {
    const float sp = fmaxf(sp_in, 0.f) + logf(1.0f + expf(-fabsf(sp_in)));
    beta[gate_row] = 1.0f / (1.0f + expf(-bv));
    g[gate_row] = -expf(decay) * sp;
  }
}

// ------------------------------------------------------------------------------------------- gather / residual add
template <typename IdT>
__global__ void __launch_bounds__(256)
embedding_gather_kernel(const IdT* ids, const __nv_bfloat16* table,
                        __nv_bfloat16* out, int tokens, int dim) {
  pdl_chain();
  const int vecs = dim >> 3;
  const int64_t total = static_cast<int64_t>(tokens) * vecs;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x; i < total; i += static_cast<int64_t>(gridDim.x) * 256) {
    const int64_t t = i / vecs;
    const int v = static_cast<int>(i % vecs);
    const int64_t id = static_cast<int64_t>(ids[t]);
    reinterpret_cast<uint4*>(out)[i] = reinterpret_cast<const uint4*>(table + id * dim)[v];
  }
}

__global__ void __launch_bounds__(256)
residual_add_kernel(const __nv_bfloat16* x, const __nv_bfloat16* r,
                    __nv_bfloat16* out, int64_t n) {
  pdl_chain();
  const int64_t vecs = n >> 3;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x; i < vecs; i += static_cast<int64_t>(gridDim.x) * 256) {
    float a[8], b[8], o[8];
    unpack8g(reinterpret_cast<const uint4*>(x)[i], a);
    unpack8g(reinterpret_cast<const uint4*>(r)[i], b);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = a[j] + b[j];
    reinterpret_cast<uint4*>(out)[i] = pack8g(o);
  }
  if (blockIdx.x == 0 && threadIdx.x < (n & 7)) {  // ragged tail
    const int64_t i = (vecs << 3) + threadIdx.x;
    out[i] = __float2bfloat16_rn(__bfloat162float(x[i]) + __bfloat162float(r[i]));
  }
}

static int grid_for(int64_t work_items, int per_block) {
  int64_t blocks = (work_items + per_block - 1) / per_block;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
  if (blocks > cap) blocks = cap;
  return static_cast<int>(blocks < 1 ? 1 : blocks);
}

}  // namespace b200

using namespace b200;

extern "C" int b200_conv4_prefill(const void* x, int64_t x_stride_t, const void* weight, int64_t w_stride_d,
                                  int64_t w_stride_k, const int32_t* seq_start, void* out, int64_t out_stride_t,
                                  int32_t tokens, int32_t channels, b200_stream_t stream) {
  B200_REQUIRE(tokens > 0 && channels > 0 && channels % 8 == 0, "conv4_prefill: channels must be a multiple of 8 (got %d)",
               channels);
  B200_REQUIRE(aligned16(x) && aligned16(out) && x_stride_t % 8 == 0 && out_stride_t % 8 == 0,
               "conv4_prefill: x and out must be 16-byte aligned with row strides that are multiples of 8 elements");
  const dim3 grid((tokens + CONV_TOKENS - 1) / CONV_TOKENS, (channels / 8 + 31) / 32);
  B200_REQUIRE(grid.y <= 65535, "conv4_prefill: too many channels (%d)", channels);
  conv4_prefill_kernel<<<grid, CONV_THREADS, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), x_stride_t, static_cast<const __nv_bfloat16*>(weight), w_stride_d, w_stride_k,
      seq_start, static_cast<__nv_bfloat16*>(out), out_stride_t, tokens, channels);
  return check_launch("conv4_prefill");
}

extern "C" int b200_conv4_decode(const void* x, int64_t x_stride_b, void* state, const void* weight4, void* out,
                                 int64_t out_stride_b, int32_t batch, int32_t channels, b200_stream_t stream) {
  B200_REQUIRE(batch > 0 && channels > 0 && channels % 8 == 0, "conv4_decode: channels must be a multiple of 8 (got %d)",
               channels);
  B200_REQUIRE(aligned16(x) && aligned16(state) && aligned16(weight4) && aligned16(out) && x_stride_b % 8 == 0 &&
                   out_stride_b % 8 == 0,
               "conv4_decode: pointers must be 16-byte aligned with row strides that are multiples of 8 elements");
  const dim3 grid(batch, (channels / 8 + CONV_THREADS - 1) / CONV_THREADS);
  B200_REQUIRE(grid.y <= 65535, "conv4_decode: too many channels (%d)", channels);
  launch_pdl(chain_overlap(), conv4_decode_kernel, dim3(grid), dim3(CONV_THREADS), 0, reinterpret_cast<cudaStream_t>(stream),
             
      static_cast<const __nv_bfloat16*>(x), x_stride_b, static_cast<__nv_bfloat16*>(state),
      static_cast<const __nv_bfloat16*>(weight4), static_cast<__nv_bfloat16*>(out), out_stride_b, channels);
  return check_launch("conv4_decode");
}

extern "C" int b200_conv_state_from_packed_prefill(void* state, const void* x, int64_t x_stride_t,
                                                   const int32_t* cu_seqlens, int32_t batch, int32_t channels,
                                                   b200_stream_t stream) {
  B200_REQUIRE(batch > 0 && channels > 0 && channels % 8 == 0,
               "conv_state_from_packed_prefill: channels must be a multiple of 8 (got %d)", channels);
  B200_REQUIRE(aligned16(x) && aligned16(state) && x_stride_t % 8 == 0,
               "conv_state_from_packed_prefill: pointers must be 16-byte aligned, the row stride a multiple of 8");
  const dim3 grid(batch, (channels / 8 + CONV_THREADS - 1) / CONV_THREADS);
  B200_REQUIRE(grid.y <= 65535, "conv_state_from_packed_prefill: too many channels (%d)", channels);
  conv_state_pack_kernel<<<grid, CONV_THREADS, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16*>(state), static_cast<const __nv_bfloat16*>(x), x_stride_t, cu_seqlens, channels);
  return check_launch("conv_state_from_packed_prefill");
}

extern "C" int b200_gdn_qk_norm_gates(const void* q, int64_t q_stride_t, int64_t q_stride_h, const void* k,
                                      int64_t k_stride_t, int64_t k_stride_h, const void* a, int64_t a_stride_t,
                                      const void* b, int64_t b_stride_t, const float* a_log, const void* dt_bias,
                                      void* q_out, void* k_out, float* beta, float* g, int32_t tokens,
                                      int32_t num_heads, int32_t head_dim, b200_stream_t stream) {
  B200_REQUIRE(tokens > 0 && num_heads > 0 && head_dim == GDN_D, "gdn_qk_norm_gates: head_dim must be %d (got %d)", GDN_D,
               head_dim);
  B200_REQUIRE((reinterpret_cast<uintptr_t>(q) % 8 == 0) && (reinterpret_cast<uintptr_t>(k) % 8 == 0) &&
                   (reinterpret_cast<uintptr_t>(q_out) % 8 == 0) && (reinterpret_cast<uintptr_t>(k_out) % 8 == 0) &&
                   q_stride_t % 4 == 0 && q_stride_h % 4 == 0 && k_stride_t % 4 == 0 && k_stride_h % 4 == 0,
               "gdn_qk_norm_gates: q, k and the outputs must be 8-byte aligned with strides that are multiples of 4");
  const int64_t rows = static_cast<int64_t>(tokens) * num_heads;
  const bool wide = rows >= GLUE_WIDE_ROWS && aligned16(q) && aligned16(k) && aligned16(q_out) && aligned16(k_out) &&
                    q_stride_t % 8 == 0 && q_stride_h % 8 == 0 && k_stride_t % 8 == 0 && k_stride_h % 8 == 0;
  const auto kernel = wide ? gdn_qk_norm_gates_wide_kernel : gdn_qk_norm_gates_kernel;
  const int per_cta = wide ? 8 : 4;
  launch_pdl(chain_overlap(), kernel, dim3(static_cast<unsigned>((rows + per_cta - 1) / per_cta)), dim3(128), 0,
             reinterpret_cast<cudaStream_t>(stream),
      static_cast<const __nv_bfloat16*>(q), q_stride_t, q_stride_h, static_cast<const __nv_bfloat16*>(k), k_stride_t,
      k_stride_h, static_cast<const __nv_bfloat16*>(a), a_stride_t, static_cast<const __nv_bfloat16*>(b), b_stride_t,
      a_log, static_cast<const __nv_bfloat16*>(dt_bias), static_cast<__nv_bfloat16*>(q_out),
      static_cast<__nv_bfloat16*>(k_out), beta, g, rows, num_heads);
  return check_launch("gdn_qk_norm_gates");
}

extern "C" int b200_embedding_gather(const void* ids, int32_t ids_are_int64, const void* table, void* out,
                                     int32_t tokens, int32_t dim, b200_stream_t stream) {
  B200_REQUIRE(tokens > 0 && dim > 0 && dim % 8 == 0 && aligned16(table) && aligned16(out),
               "embedding_gather: dim must be a multiple of 8 (got %d), table and out 16-byte aligned", dim);
  const int blocks = grid_for(static_cast<int64_t>(tokens) * (dim / 8), 256);
  if (ids_are_int64)
    launch_pdl(chain_overlap(), embedding_gather_kernel<int64_t>, dim3(blocks), dim3(256), 0, reinterpret_cast<cudaStream_t>(stream),
             
        static_cast<const int64_t*>(ids), static_cast<const __nv_bfloat16*>(table), static_cast<__nv_bfloat16*>(out),
        tokens, dim);
  else
    launch_pdl(chain_overlap(), embedding_gather_kernel<int32_t>, dim3(blocks), dim3(256), 0, reinterpret_cast<cudaStream_t>(stream),
             
        static_cast<const int32_t*>(ids), static_cast<const __nv_bfloat16*>(table), static_cast<__nv_bfloat16*>(out),
        tokens, dim);
  return check_launch("embedding_gather");
}

extern "C" int b200_residual_add(const void* x, const void* residual, void* out, int64_t count, b200_stream_t stream) {
  B200_REQUIRE(count > 0 && aligned16(x) && aligned16(residual) && aligned16(out),
               "residual_add: pointers must be 16-byte aligned");
  launch_pdl(chain_overlap(), residual_add_kernel, dim3(grid_for(count / 8 + 1, 256)), dim3(256), 0, reinterpret_cast<cudaStream_t>(stream),
             
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(residual), static_cast<__nv_bfloat16*>(out),
      count);
  return check_launch("residual_add");
}
