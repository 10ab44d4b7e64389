// Row-wise operators between the projections and the attention / Gated-DeltaNet kernels of a layer, each one launch
// where the reference spends one to three and an eager PyTorch restatement a dozen:
//   b200_add_rmsnorm        <-> triton_kernels/residual_add.py + triton_kernels/qwen_rmsnorm.py:70-73
//   b200_swiglu             <-> triton_kernels/swiglu.py
//   b200_gdn_decode_prep    <-> triton_kernels/depthwise_causal_conv4_decode.py + triton_kernels/gdn_qk_norm_gates.py:68-89
//   b200_gdn_gated_rmsnorm  <-> triton_kernels/gdn_gated_rmsnorm.py:54-67
//   b200_argmax_rows        <-> the arg-max half of triton_kernels/vocab_argmax.py:141-200 (fp32 logits in, ids out)
// All are HBM/launch bound: 16-byte accesses, one warp per row (or one CTA per (sequence, head)), fp32 math, one
// rounding to bf16 at the reference's rounding points.
#include "b200_attn.h"
#include "common.cuh"

namespace b200 {

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  f[0] = bf16_lo(v.x); f[1] = bf16_hi(v.x); f[2] = bf16_lo(v.y); f[3] = bf16_hi(v.y);
  f[4] = bf16_lo(v.z); f[5] = bf16_hi(v.z); f[6] = bf16_lo(v.w); f[7] = bf16_hi(v.w);
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  return make_uint4(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]), pack_bf16(f[4], f[5]), pack_bf16(f[6], f[7]));
}

// ------------------------------------------------------------------------------------------ (residual +) RMSNorm
// CTA = one row, thread = 8 consecutive elements (blockDim = dim / 8, a multiple of 32): every global load of a
// thread is issued before the first use, so a call costs one memory round trip plus the block reduction.
constexpr int RN_MAX_DIM = 8192;

__global__ void __launch_bounds__(RN_MAX_DIM / 8)
add_rmsnorm_kernel(const __nv_bfloat16* x, int64_t x_outer, int64_t x_inner, int inner_count,  // x, residual: no
                   const __nv_bfloat16* residual, int64_t res_stride,                             // __restrict__ (pdl_wait)
                   const __nv_bfloat16* __restrict__ weight, __nv_bfloat16* __restrict__ sum_out,
                   __nv_bfloat16* __restrict__ norm_out, int dim, float eps, int overlap) {
  __shared__ float red[32];
  const int row = blockIdx.x, c = threadIdx.x * 8;
  const __nv_bfloat16* src = x + static_cast<int64_t>(row / inner_count) * x_outer + (row % inner_count) * x_inner;
  if (overlap & OVERLAP_TRIGGER) pdl_trigger();
  const uint4 wv = *reinterpret_cast<const uint4*>(weight + c);  // a weight: independent of the predecessor
  pdl_wait();
  const uint4 xv = *reinterpret_cast<const uint4*>(src + c);
  uint4 rv = make_uint4(0, 0, 0, 0);
  if (residual != nullptr) rv = *reinterpret_cast<const uint4*>(residual + static_cast<int64_t>(row) * res_stride + c);
  float v[8], w[8];
  unpack8(xv, v);
  unpack8(wv, w);
  if (residual != nullptr) {
    float r[8];
    unpack8(rv, r);
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = round_bf16(v[j] + r[j]);  // the sum is a bf16 tensor in the reference
    if (sum_out != nullptr) *reinterpret_cast<uint4*>(sum_out + static_cast<int64_t>(row) * dim + c) = pack8(v);
  }
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) ss = fmaf(v[j], v[j], ss);
  ss = warp_sum(ss);
  const int warps = blockDim.x >> 5;
  if (warps > 1) {
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    ss = 0.f;
    for (int i = 0; i < warps; ++i) ss += red[i];
  }
  const float rs = rsqrtf(ss / static_cast<float>(dim) + eps);
  float o[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) o[j] = v[j] * rs * (1.0f + w[j]);
  *reinterpret_cast<uint4*>(norm_out + static_cast<int64_t>(row) * dim + c) = pack8(o);
}

// Prompt-sized form: one warp per row, four rows per CTA, lane = VPL 16-byte vectors 32 vectors apart (dim = VPL * 256);
// no shared memory and no block barrier, and a CTA keeps up to 12 * VPL loads per lane in flight.
template <int VPL>
__global__ void __launch_bounds__(128)
add_rmsnorm_rows_kernel(const __nv_bfloat16* x, int64_t x_outer, int64_t x_inner, int inner_count,
                        const __nv_bfloat16* residual, int64_t res_stride,
                        const __nv_bfloat16* __restrict__ weight, __nv_bfloat16* __restrict__ sum_out,
                        __nv_bfloat16* __restrict__ norm_out, int rows, float eps, int overlap) {
  constexpr int DIM = VPL * 256;
  const int row = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (overlap & OVERLAP_TRIGGER) pdl_trigger();
  uint4 wv[VPL];
#pragma unroll
  for (int j = 0; j < VPL; ++j) wv[j] = *reinterpret_cast<const uint4*>(weight + (lane + 32 * j) * 8);
  pdl_wait();
  if (row >= rows) return;
  const __nv_bfloat16* src = x + static_cast<int64_t>(row / inner_count) * x_outer + (row % inner_count) * x_inner;
  uint4 xv[VPL], rv[VPL];
#pragma unroll
  for (int j = 0; j < VPL; ++j) xv[j] = *reinterpret_cast<const uint4*>(src + (lane + 32 * j) * 8);
  if (residual != nullptr) {
#pragma unroll
    for (int j = 0; j < VPL; ++j)
      rv[j] = *reinterpret_cast<const uint4*>(residual + static_cast<int64_t>(row) * res_stride + (lane + 32 * j) * 8);
  }
  float v[VPL][8];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < VPL; ++j) {
    unpack8(xv[j], v[j]);
    if (residual != nullptr) {
      float r[8];
      unpack8(rv[j], r);
#pragma unroll
      for (int e = 0; e < 8; ++e) v[j][e] = round_bf16(v[j][e] + r[e]);  // the sum is a bf16 tensor in the reference
      if (sum_out != nullptr)
        *reinterpret_cast<uint4*>(sum_out + static_cast<int64_t>(row) * DIM + (lane + 32 * j) * 8) = pack8(v[j]);
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) ss = fmaf(v[j][e], v[j][e], ss);
  }
  ss = warp_sum(ss);
  const float rs = rsqrtf(ss / static_cast<float>(DIM) + eps);
#pragma unroll
  for (int j = 0; j < VPL; ++j) {
    float w[8], o[8];
    unpack8(wv[j], w);
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = v[j][e] * rs * (1.0f + w[e]);
    *reinterpret_cast<uint4*>(norm_out + static_cast<int64_t>(row) * DIM + (lane + 32 * j) * 8) = pack8(o);
  }
}

// ------------------------------------------------------------------------------------------------------- SwiGLU
__global__ void __launch_bounds__(256)
swiglu_kernel(const __nv_bfloat16* gate, int64_t gate_stride, const __nv_bfloat16* up, int64_t up_stride,
              __nv_bfloat16* __restrict__ out, int rows, int inter, int overlap) {
  const int vec_per_row = inter >> 3;
  const int64_t total = static_cast<int64_t>(rows) * vec_per_row;
  if (overlap & OVERLAP_TRIGGER) pdl_trigger();
  pdl_wait();
  for (int64_t idx = blockIdx.x * 256 + threadIdx.x; idx < total; idx += static_cast<int64_t>(gridDim.x) * 256) {
    const int64_t r = idx / vec_per_row;
    const int c = static_cast<int>(idx % vec_per_row) * 8;
    float g[8], u[8], o[8];
    unpack8(*reinterpret_cast<const uint4*>(gate + r * gate_stride + c), g);
    unpack8(*reinterpret_cast<const uint4*>(up + r * up_stride + c), u);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = g[j] / (1.0f + expf(-g[j])) * u[j];
    *reinterpret_cast<uint4*>(out + r * inter + c) = pack8(o);
  }
}

// Prompt-sized form: thread = one 8-wide column vector of SW_ROWS consecutive rows, every load issued before the first
// use; no index division; fast exponential and reciprocal.
constexpr int SW_ROWS = 4;
constexpr int SW_THREADS = 64;

__global__ void __launch_bounds__(SW_THREADS)
swiglu_rows_kernel(const __nv_bfloat16* gate, int64_t gate_stride, const __nv_bfloat16* up, int64_t up_stride,
                   __nv_bfloat16* __restrict__ out, int rows, int inter, int overlap) {
  if (overlap & OVERLAP_TRIGGER) pdl_trigger();
  pdl_wait();
  const int c = (blockIdx.x * SW_THREADS + threadIdx.x) * 8;
  if (c >= inter) return;
  const int r0 = blockIdx.y * SW_ROWS;
  uint4 gv[SW_ROWS], uv[SW_ROWS];
#pragma unroll
  for (int j = 0; j < SW_ROWS; ++j) {
    const int64_t r = min(r0 + j, rows - 1);
    gv[j] = *reinterpret_cast<const uint4*>(gate + r * gate_stride + c);
    uv[j] = *reinterpret_cast<const uint4*>(up + r * up_stride + c);
  }
#pragma unroll
  for (int j = 0; j < SW_ROWS; ++j) {
    if (r0 + j >= rows) break;
    float g[8], u[8], o[8];
    unpack8(gv[j], g);
    unpack8(uv[j], u);
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = silu_fast(g[e]) * u[e];
    *reinterpret_cast<uint4*>(out + static_cast<int64_t>(r0 + j) * inter + c) = pack8(o);
  }
}

// ------------------------------------------------------------------------------- GDN decode: conv + norms + gates
// CTA = (head, sequence), thread t = channel t of the head's q, k and v slices of the [3*H*128] conv width.
__global__ void __launch_bounds__(GDN_D)
gdn_decode_prep_kernel(const __nv_bfloat16* qkv, int64_t qkv_stride, __nv_bfloat16* conv_state,
                       const __nv_bfloat16* w4, const __nv_bfloat16* a, int64_t a_stride,
                       const __nv_bfloat16* b, int64_t b_stride, const float* a_log,
                       const __nv_bfloat16* dt_bias, __nv_bfloat16* q_out,
                       __nv_bfloat16* k_out, __nv_bfloat16* v_out, float* beta,
                       float* g, int heads) {
  pdl_chain();
  __shared__ float red[2][4];
  const int h = blockIdx.x, seq = blockIdx.y, t = threadIdx.x;
  const int width = 3 * heads * GDN_D;
  float y[3];
#pragma unroll
  for (int part = 0; part < 3; ++part) {
    const int c = part * heads * GDN_D + h * GDN_D + t;
    __nv_bfloat16* st = conv_state + static_cast<int64_t>(seq) * 4 * width + c;
    const __nv_bfloat16 s1 = st[width], s2 = st[2 * width], s3 = st[3 * width];
    const __nv_bfloat16 xn = qkv[static_cast<int64_t>(seq) * qkv_stride + c];
    st[0] = s1;
    st[width] = s2;
    st[2 * width] = s3;
    st[3 * width] = xn;
    float acc = __bfloat162float(w4[c]) * __bfloat162float(s1);
    acc = fmaf(__bfloat162float(w4[width + c]), __bfloat162float(s2), acc);
    acc = fmaf(__bfloat162float(w4[2 * width + c]), __bfloat162float(s3), acc);
    acc = fmaf(__bfloat162float(w4[3 * width + c]), __bfloat162float(xn), acc);
    y[part] = round_bf16(acc / (1.0f + expf(-acc)));  // the conv output is a bf16 tensor in the reference
  }
  float sq = warp_sum(y[0] * y[0]), sk = warp_sum(y[1] * y[1]);
  if ((t & 31) == 0) {
    red[0][t >> 5] = sq;
    red[1][t >> 5] = sk;
  }
  __syncthreads();
  sq = (red[0][0] + red[0][1]) + (red[0][2] + red[0][3]);
  sk = (red[1][0] + red[1][1]) + (red[1][2] + red[1][3]);
  const int64_t o = (static_cast<int64_t>(seq) * heads + h) * GDN_D + t;
  q_out[o] = __float2bfloat16_rn(y[0] * rsqrtf(sq + 1e-6f) * 0.08838834764831845f);  // DK^-0.5, DK = 128
  k_out[o] = __float2bfloat16_rn(y[1] * rsqrtf(sk + 1e-6f));
  v_out[o] = __float2bfloat16_rn(y[2]);
  if (t == 0) {
    const float av = __bfloat162float(a[static_cast<int64_t>(seq) * a_stride + h]) + __bfloat162float(dt_bias[h]);
    const float bv = __bfloat162float(b[static_cast<int64_t>(seq) * b_stride + h]);
    const float sp = av > 20.f ? av : log1pf(expf(av));
    beta[static_cast<int64_t>(seq) * heads + h] = 1.0f / (1.0f + expf(-bv));
    g[static_cast<int64_t>(seq) * heads + h] = -expf(a_log[h]) * sp;
  }
}

// ------------------------------------------------------------------------------------------- gated RMSNorm (GDN)
__global__ void __launch_bounds__(128)
gdn_gated_rmsnorm_kernel(const __nv_bfloat16* x, const __nv_bfloat16* z, int64_t z_stride,
                         const float* weight, __nv_bfloat16* out, int rows, int heads) {
  pdl_chain();
  const int row = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= rows) return;
  const int n = row / heads, h = row % heads;
  const uint2 xv = *reinterpret_cast<const uint2*>(x + static_cast<int64_t>(row) * GDN_D + lane * 4);
  const uint2 zv = *reinterpret_cast<const uint2*>(z + static_cast<int64_t>(n) * z_stride + h * GDN_D + lane * 4);
  const float4 wv = *reinterpret_cast<const float4*>(weight + lane * 4);
  const float xf[4] = {bf16_lo(xv.x), bf16_hi(xv.x), bf16_lo(xv.y), bf16_hi(xv.y)};
  const float zf[4] = {bf16_lo(zv.x), bf16_hi(zv.x), bf16_lo(zv.y), bf16_hi(zv.y)};
  const float wf[4] = {wv.x, wv.y, wv.z, wv.w};
  const float ss = warp_sum((xf[0] * xf[0] + xf[1] * xf[1]) + (xf[2] * xf[2] + xf[3] * xf[3]));
  const float rs = rsqrtf(ss / static_cast<float>(GDN_D) + 1e-6f);
  float o[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) o[j] = xf[j] * rs * wf[j] * (zf[j] / (1.0f + expf(-zf[j])));
  *reinterpret_cast<uint2*>(out + static_cast<int64_t>(row) * GDN_D + lane * 4) =
      make_uint2(pack_bf16(o[0], o[1]), pack_bf16(o[2], o[3]));
}

// Prompt-sized form (16-byte aligned rows): 16 lanes x 8 elements per row, eight rows per CTA, fast SiLU.
__global__ void __launch_bounds__(128)
gdn_gated_rmsnorm_wide_kernel(const __nv_bfloat16* x, const __nv_bfloat16* z, int64_t z_stride,
                              const float* weight, __nv_bfloat16* out, int rows, int heads) {
  pdl_chain();
  const int sub = threadIdx.x & 15;
  const int row_raw = blockIdx.x * 8 + (threadIdx.x >> 4);
  const bool live = row_raw < rows;
  const int row = live ? row_raw : rows - 1;  // a dead half-warp repeats the last row and stores nothing
  const int n = row / heads, h = row % heads;
  const uint4 xv = *reinterpret_cast<const uint4*>(x + static_cast<int64_t>(row) * GDN_D + sub * 8);
  const uint4 zv = *reinterpret_cast<const uint4*>(z + static_cast<int64_t>(n) * z_stride + h * GDN_D + sub * 8);
  const float4 w0 = *reinterpret_cast<const float4*>(weight + sub * 8);
  const float4 w1 = *reinterpret_cast<const float4*>(weight + sub * 8 + 4);
  const float wf[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
  float xf[8], zf[8], o[8];
  unpack8(xv, xf);
  unpack8(zv, zf);
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) ss = fmaf(xf[j], xf[j], ss);
#pragma unroll
  for (int s = 8; s > 0; s >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, s);
  const float rs = rsqrtf(ss / static_cast<float>(GDN_D) + 1e-6f);
#pragma unroll
  for (int j = 0; j < 8; ++j) o[j] = xf[j] * rs * wf[j] * silu_fast(zf[j]);
  if (live) *reinterpret_cast<uint4*>(out + static_cast<int64_t>(row) * GDN_D + sub * 8) = pack8(o);
}

// ------------------------------------------------------------------------------------------- row arg-max (LM head)
// ids[r] = argmax_n logits[r, n], ties to the lowest n (triton_kernels/vocab_argmax.py:141-200).  A (value, index)
// pair is packed into one 64-bit key whose unsigned order is "larger value first, then smaller index"; a CTA reduces
// one slice of one row (16-byte loads, every thread walks its elements in ascending order), the slices of a row meet
// in an atomicMax, and the last slice to arrive (a counter per row) unpacks the index and leaves key and counter zero
// for the next launch.
constexpr int AM_THREADS = 256;
constexpr int AM_MAX_ROWS = 1024;

__global__ void __launch_bounds__(AM_THREADS)
argmax_rows_kernel(const float* logits, int64_t row_stride, int n, int64_t* __restrict__ ids,  // logits: no __restrict__
                   unsigned long long* keys, int* counters, int overlap) {                    // (read after pdl_wait)
  __shared__ unsigned long long red[AM_THREADS / 32];
  const int row = blockIdx.y, splits = gridDim.x;
  const int vecs = n >> 2;                                       // n is a multiple of 4
  const int per = (vecs + splits - 1) / splits;
  const int v0 = blockIdx.x * per, v1 = min(v0 + per, vecs);
  pdl_wait();
  const float4* src = reinterpret_cast<const float4*>(logits + static_cast<int64_t>(row) * row_stride);
  float best = -INFINITY;
  uint32_t best_i = 0xffffffffu;                                 // "nothing yet": loses every tie
  for (int i = v0 + threadIdx.x; i < v1; i += AM_THREADS) {
    const float4 x = __ldcs(src + i);
    const uint32_t base = static_cast<uint32_t>(i) * 4u;
    // strict > keeps the first of equal values inside this thread's ascending walk; NaN compares false and is skipped
    if (x.x > best || best_i == 0xffffffffu) { best = x.x; best_i = base; }
    if (x.y > best) { best = x.y; best_i = base + 1; }
    if (x.z > best) { best = x.z; best_i = base + 2; }
    if (x.w > best) { best = x.w; best_i = base + 3; }
  }
  unsigned long long key = best_i == 0xffffffffu ? 0ull : argmax_key(best, best_i);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const unsigned long long other = __shfl_xor_sync(0xffffffffu, key, o);
    key = other > key ? other : key;
  }
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = key;
  __syncthreads();
  if (threadIdx.x == 0) {
#pragma unroll
    for (int w = 1; w < AM_THREADS / 32; ++w) key = red[w] > key ? red[w] : key;
    atomicMax(keys + row, key);
    __threadfence();
    if (atomicAdd(counters + row, 1) == splits - 1) {
      __threadfence();
      const unsigned long long top = atomicExch(keys + row, 0ull);
      ids[row] = static_cast<int64_t>(0xffffffffu - static_cast<uint32_t>(top & 0xffffffffull));
      counters[row] = 0;
    }
  }
}

}  // namespace b200

using namespace b200;

extern "C" int b200_add_rmsnorm(const void* x, int64_t x_stride_outer, int64_t x_stride_inner, int32_t inner_count,
                                const void* residual, int64_t residual_stride, const void* weight, void* sum_out,
                                void* norm_out, int32_t rows, int32_t dim, float eps, int32_t overlap, b200_stream_t stream) {
  B200_REQUIRE(rows > 0 && inner_count > 0 && dim > 0 && dim % 256 == 0 && dim <= RN_MAX_DIM,
               "add_rmsnorm: dim must be a multiple of 256 up to %d (got %d)", RN_MAX_DIM, dim);
  B200_REQUIRE(aligned16(x) && aligned16(weight) && aligned16(norm_out) && x_stride_outer % 8 == 0 &&
                   x_stride_inner % 8 == 0,
               "add_rmsnorm: pointers must be 16-byte aligned and row strides multiples of 8 elements");
  B200_REQUIRE(residual == nullptr || (aligned16(residual) && residual_stride % 8 == 0 &&
                                       (sum_out == nullptr || aligned16(sum_out))),
               "add_rmsnorm: residual / sum_out must be 16-byte aligned with a row stride that is a multiple of 8");
  if (rows >= GLUE_WIDE_ROWS && (dim == 256 || dim == 512 || dim == 1024 || dim == 2048)) {
    const auto kernel = dim == 256 ? add_rmsnorm_rows_kernel<1> : dim == 512 ? add_rmsnorm_rows_kernel<2>
                      : dim == 1024 ? add_rmsnorm_rows_kernel<4> : add_rmsnorm_rows_kernel<8>;
    if (launch_pdl((overlap & OVERLAP_START) != 0, kernel, dim3((rows + 3) / 4), dim3(128), 0,
                   reinterpret_cast<cudaStream_t>(stream), static_cast<const __nv_bfloat16*>(x), x_stride_outer,
                   x_stride_inner, inner_count, static_cast<const __nv_bfloat16*>(residual), residual_stride,
                   static_cast<const __nv_bfloat16*>(weight), static_cast<__nv_bfloat16*>(sum_out),
                   static_cast<__nv_bfloat16*>(norm_out), rows, eps, overlap) != cudaSuccess)
      return fail(ERR_LAUNCH, "add_rmsnorm: %s", cudaGetErrorString(cudaGetLastError()));
    return check_launch("add_rmsnorm");
  }
  if (launch_pdl((overlap & OVERLAP_START) != 0, add_rmsnorm_kernel, dim3(rows), dim3(dim / 8), 0, reinterpret_cast<cudaStream_t>(stream),
                 static_cast<const __nv_bfloat16*>(x), x_stride_outer, x_stride_inner, inner_count,
                 static_cast<const __nv_bfloat16*>(residual), residual_stride, static_cast<const __nv_bfloat16*>(weight),
                 static_cast<__nv_bfloat16*>(sum_out), static_cast<__nv_bfloat16*>(norm_out), dim, eps, overlap) != cudaSuccess)
    return fail(ERR_LAUNCH, "add_rmsnorm: %s", cudaGetErrorString(cudaGetLastError()));
  return check_launch("add_rmsnorm");
}

// Decode-sized calls take the flat one-vector-per-thread kernel, prompt-sized ones the row-blocked kernel.
static cudaError_t launch_swiglu(bool start_early, const __nv_bfloat16* gate, int64_t gate_stride, const __nv_bfloat16* up,
                                 int64_t up_stride, __nv_bfloat16* out, int rows, int width, int overlap,
                                 b200_stream_t stream) {
  const int row_blocks = (rows + SW_ROWS - 1) / SW_ROWS;
  if (rows >= GLUE_WIDE_ROWS && row_blocks <= 65535)
    return launch_pdl(start_early, swiglu_rows_kernel, dim3((width / 8 + SW_THREADS - 1) / SW_THREADS, row_blocks),
                      dim3(SW_THREADS), 0, reinterpret_cast<cudaStream_t>(stream), gate, gate_stride, up, up_stride, out,
                      rows, width, overlap);
  const int64_t vecs = static_cast<int64_t>(rows) * (width / 8);
  int blocks = static_cast<int>((vecs + 255) / 256);
  const int cap = sm_count() * 8;
  if (blocks > cap) blocks = cap;
  return launch_pdl(start_early, swiglu_kernel, dim3(blocks), dim3(256), 0, reinterpret_cast<cudaStream_t>(stream), gate,
                    gate_stride, up, up_stride, out, rows, width, overlap);
}

extern "C" int b200_swiglu(const void* gate_up, int64_t row_stride, void* out, int32_t rows, int32_t intermediate,
                           int32_t overlap, b200_stream_t stream) {
  B200_REQUIRE(rows > 0 && intermediate > 0 && intermediate % 8 == 0 && row_stride % 8 == 0 && aligned16(gate_up) &&
                   aligned16(out),
               "swiglu: intermediate and the row stride must be multiples of 8, pointers 16-byte aligned");
  if (launch_swiglu((overlap & OVERLAP_START) != 0, static_cast<const __nv_bfloat16*>(gate_up), row_stride,
                    static_cast<const __nv_bfloat16*>(gate_up) + intermediate, row_stride,
                    static_cast<__nv_bfloat16*>(out), rows, intermediate, overlap, stream) != cudaSuccess)
    return fail(ERR_LAUNCH, "swiglu: %s", cudaGetErrorString(cudaGetLastError()));
  return check_launch("swiglu");
}

extern "C" int b200_swiglu_pair(const void* gate, int64_t gate_stride, const void* up, int64_t up_stride, void* out,
                                int32_t rows, int32_t width, b200_stream_t stream) {
  B200_REQUIRE(rows > 0 && width > 0 && width % 8 == 0 && gate_stride % 8 == 0 && up_stride % 8 == 0 && aligned16(gate) &&
                   aligned16(up) && aligned16(out),
               "swiglu_pair: the width and the row strides must be multiples of 8, pointers 16-byte aligned");
  const bool chain = chain_overlap();
  if (launch_swiglu(chain, static_cast<const __nv_bfloat16*>(gate), gate_stride, static_cast<const __nv_bfloat16*>(up),
                    up_stride, static_cast<__nv_bfloat16*>(out), rows, width, chain ? OVERLAP_TRIGGER : 0,
                    stream) != cudaSuccess)
    return fail(ERR_LAUNCH, "swiglu_pair: %s", cudaGetErrorString(cudaGetLastError()));
  return check_launch("swiglu_pair");
}

extern "C" int b200_gdn_decode_prep(const void* qkv, int64_t qkv_stride, void* conv_state, const void* weight4,
                                    const void* a, int64_t a_stride, const void* b, int64_t b_stride,
                                    const float* a_log, const void* dt_bias, void* q_out, void* k_out, void* v_out,
                                    float* beta, float* g, int32_t batch, int32_t num_heads, int32_t head_dim,
                                    b200_stream_t stream) {
  B200_REQUIRE(batch > 0 && batch <= 65535 && num_heads > 0 && head_dim == GDN_D,
               "gdn_decode_prep: head_dim must be %d (got %d)", GDN_D, head_dim);
  launch_pdl(chain_overlap(), gdn_decode_prep_kernel, dim3(num_heads, batch), dim3(GDN_D), 0, reinterpret_cast<cudaStream_t>(stream),
             
      static_cast<const __nv_bfloat16*>(qkv), qkv_stride, static_cast<__nv_bfloat16*>(conv_state),
      static_cast<const __nv_bfloat16*>(weight4), static_cast<const __nv_bfloat16*>(a), a_stride,
      static_cast<const __nv_bfloat16*>(b), b_stride, a_log, static_cast<const __nv_bfloat16*>(dt_bias),
      static_cast<__nv_bfloat16*>(q_out), static_cast<__nv_bfloat16*>(k_out), static_cast<__nv_bfloat16*>(v_out), beta, g,
      num_heads);
  return check_launch("gdn_decode_prep");
}

extern "C" int b200_gdn_gated_rmsnorm(const void* x, const void* z, int64_t z_stride, const float* weight, void* out,
                                      int32_t rows, int32_t num_heads, int32_t head_dim, b200_stream_t stream) {
  B200_REQUIRE(rows > 0 && num_heads > 0 && head_dim == GDN_D, "gdn_gated_rmsnorm: head_dim must be %d (got %d)", GDN_D,
               head_dim);
  B200_REQUIRE(z_stride % 4 == 0 && (reinterpret_cast<uintptr_t>(x) % 8 == 0) && (reinterpret_cast<uintptr_t>(z) % 8 == 0) &&
                   (reinterpret_cast<uintptr_t>(out) % 8 == 0) && aligned16(weight),
               "gdn_gated_rmsnorm: x, z, out must be 8-byte aligned, weight 16-byte aligned, z stride a multiple of 4");
  const bool wide = rows >= GLUE_WIDE_ROWS && z_stride % 8 == 0 && aligned16(x) && aligned16(z) && aligned16(out);
  launch_pdl(chain_overlap(), wide ? gdn_gated_rmsnorm_wide_kernel : gdn_gated_rmsnorm_kernel,
             dim3(wide ? (rows + 7) / 8 : (rows + 3) / 4), dim3(128), 0, reinterpret_cast<cudaStream_t>(stream),
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(z), z_stride, weight,
      static_cast<__nv_bfloat16*>(out), rows, num_heads);
  return check_launch("gdn_gated_rmsnorm");
}

extern "C" int64_t b200_argmax_rows_workspace_bytes(void) { return AM_MAX_ROWS * (8 + 4); }

extern "C" int b200_argmax_rows(const float* logits, int64_t row_stride, int64_t* ids, void* workspace, int32_t rows,
                                int32_t n, int32_t overlap, b200_stream_t stream) {
  B200_REQUIRE(rows > 0 && rows <= AM_MAX_ROWS && n > 0 && n % 4 == 0 && row_stride % 4 == 0,
               "argmax_rows: rows must be in [1, %d], n and the row stride multiples of 4 (got %d rows, n=%d)", AM_MAX_ROWS,
               rows, n);
  B200_REQUIRE(aligned16(logits) && workspace != nullptr && (reinterpret_cast<uintptr_t>(workspace) % 8 == 0) &&
                   ids != nullptr,
               "argmax_rows: logits must be 16-byte aligned, the workspace 8-byte aligned");
  // slices of at least 8192 elements; enough CTAs to fill the machine for a decode batch
  int splits = sm_count() * 2 / rows;
  const int max_splits = (n / 4 + 2047) / 2048;
  if (splits > max_splits) splits = max_splits;
  if (splits < 1) splits = 1;
  unsigned long long* keys = static_cast<unsigned long long*>(workspace);
  int* counters = reinterpret_cast<int*>(keys + AM_MAX_ROWS);
  if (launch_pdl((overlap & OVERLAP_START) != 0, argmax_rows_kernel, dim3(splits, rows), dim3(AM_THREADS), 0,
                 reinterpret_cast<cudaStream_t>(stream), logits, row_stride, n, ids, keys, counters, overlap) != cudaSuccess)
    return fail(ERR_LAUNCH, "argmax_rows: %s", cudaGetErrorString(cudaGetLastError()));
  return check_launch("argmax_rows");
}
