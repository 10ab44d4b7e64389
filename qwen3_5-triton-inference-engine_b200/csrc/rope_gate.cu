// Stand-alone partial RoPE and sigmoid gate-pack (the fused attention kernels apply both themselves; these
// entry points exist so the reference's operators of the same names have drop-in counterparts).
//   b200_partial_rope        <-> triton_kernels/partial_rope.py:27-132 (+ op :145-198)
//   b200_attention_gate_pack <-> triton_kernels/attention_gate_pack.py:15-64 (+ op :77-126)
#include "b200_attn.h"
#include "common.cuh"

namespace b200 {

// One thread per (b, h, t, column-pair or tail element).  Columns [0,R/2) pair with [R/2,R); angles are
// pos(fp32) * inv_freq in fp32 with full-range sinf/cosf (positions reach 32768 rad at inv_freq = 1).
__global__ void partial_rope_kernel(const __nv_bfloat16* x, int64_t x_b, int64_t x_h, int64_t x_t,
                                    __nv_bfloat16* out, int64_t o_b, int64_t o_h, int64_t o_t,
                                    const void* position_ids, int ids_are_int64, int64_t id_b,
                                    int64_t id_t, const float* inv_freq, int batch, int heads,
                                    int tokens, int d, int r) {
  pdl_chain();
  const int half = r / 2;
  const int per_row = half + (d - r);  // work items per (b,h,t) row
  const int64_t total = static_cast<int64_t>(batch) * heads * tokens * per_row;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>(i % per_row);
    int64_t rest = i / per_row;
    const int t = static_cast<int>(rest % tokens);
    rest /= tokens;
    const int h = static_cast<int>(rest % heads);
    const int b = static_cast<int>(rest / heads);
    const __nv_bfloat16* xr = x + b * x_b + h * x_h + t * x_t;
    __nv_bfloat16* orow = out + b * o_b + h * o_h + t * o_t;
    if (c < half) {
      const int64_t pid = ids_are_int64 ? static_cast<const int64_t*>(position_ids)[b * id_b + t * id_t]
                                        : static_cast<int64_t>(static_cast<const int32_t*>(position_ids)[b * id_b + t * id_t]);
      const float angle = static_cast<float>(pid) * inv_freq[c];
      float sn, cs;
      sincosf(angle, &sn, &cs);
      const float a = __bfloat162float(xr[c]), bb = __bfloat162float(xr[c + half]);
      float o1, o2;
      rope_pair(a, bb, sn, cs, o1, o2);
      orow[c] = __float2bfloat16_rn(o1);
      orow[c + half] = __float2bfloat16_rn(o2);
    } else {
      const int col = r + (c - half);
      orow[col] = xr[col];
    }
  }
}

// out[t, h*D + d] = bf16(x[h,t,d] * sigmoid(gate[h,t,d])) with fp32 math; 8 elements per thread when aligned.
__global__ void gate_pack_kernel(const __nv_bfloat16* x, int64_t x_h, int64_t x_t,
                                 const __nv_bfloat16* gate, int64_t g_h, int64_t g_t,
                                 __nv_bfloat16* out, int heads, int tokens, int d, int vec_ok) {
  pdl_chain();
  const int step = vec_ok ? 8 : 1;
  const int per_row = d / step;
  const int64_t total = static_cast<int64_t>(tokens) * heads * per_row;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>(i % per_row) * step;
    int64_t rest = i / per_row;
    const int h = static_cast<int>(rest % heads);
    const int t = static_cast<int>(rest / heads);
    const __nv_bfloat16* xr = x + h * x_h + t * x_t + c;
    const __nv_bfloat16* gr = gate + h * g_h + t * g_t + c;
    __nv_bfloat16* orow = out + (static_cast<int64_t>(t) * heads + h) * d + c;
    if (vec_ok) {
      const uint4 xv = *reinterpret_cast<const uint4*>(xr);
      const uint4 gv = *reinterpret_cast<const uint4*>(gr);
      const uint32_t xs[4] = {xv.x, xv.y, xv.z, xv.w}, gs[4] = {gv.x, gv.y, gv.z, gv.w};
      uint32_t os[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float lo = bf16_lo(xs[j]) * (1.f / (1.f + __expf(-bf16_lo(gs[j]))));
        const float hi = bf16_hi(xs[j]) * (1.f / (1.f + __expf(-bf16_hi(gs[j]))));
        os[j] = pack_bf16(lo, hi);
      }
      *reinterpret_cast<uint4*>(orow) = make_uint4(os[0], os[1], os[2], os[3]);
    } else {
      const float g = __bfloat162float(*gr);
      *orow = __float2bfloat16_rn(__bfloat162float(*xr) * (1.f / (1.f + __expf(-g))));
    }
  }
}

}  // namespace b200

using namespace b200;

extern "C" int b200_partial_rope(const void* x, int64_t x_stride_b, int64_t x_stride_h, int64_t x_stride_t, void* out,
                                 int64_t out_stride_b, int64_t out_stride_h, int64_t out_stride_t,
                                 const void* position_ids, int32_t ids_are_int64, int64_t ids_stride_b,
                                 int64_t ids_stride_t, const float* inv_freq, int32_t batch, int32_t num_heads,
                                 int32_t num_tokens, int32_t head_dim, int32_t rotary_dim, b200_stream_t stream) {
  B200_REQUIRE(batch > 0 && num_heads > 0 && num_tokens > 0 && head_dim > 0, "partial_rope: empty shape");
  B200_REQUIRE(rotary_dim > 0 && rotary_dim <= head_dim && rotary_dim % 2 == 0,
               "partial_rope: rotary_dim must be even and in (0, head_dim]");
  const int64_t total = static_cast<int64_t>(batch) * num_heads * num_tokens * (rotary_dim / 2 + head_dim - rotary_dim);
  const int threads = 256;
  const int64_t want = (total + threads - 1) / threads;
  const unsigned grid = static_cast<unsigned>(want < 1 ? 1 : (want > 148 * 16 ? 148 * 16 : want));
  launch_pdl(chain_overlap(), partial_rope_kernel, dim3(grid), dim3(threads), 0, reinterpret_cast<cudaStream_t>(stream),
             
      static_cast<const __nv_bfloat16*>(x), x_stride_b, x_stride_h, x_stride_t, static_cast<__nv_bfloat16*>(out),
      out_stride_b, out_stride_h, out_stride_t, position_ids, ids_are_int64, ids_stride_b, ids_stride_t, inv_freq,
      batch, num_heads, num_tokens, head_dim, rotary_dim);
  return check_launch("partial_rope");
}

extern "C" int b200_attention_gate_pack(const void* x, int64_t x_stride_h, int64_t x_stride_t, const void* gate,
                                        int64_t gate_stride_h, int64_t gate_stride_t, void* out, int32_t num_heads,
                                        int32_t num_tokens, int32_t head_dim, b200_stream_t stream) {
  B200_REQUIRE(num_heads > 0 && num_tokens > 0 && head_dim > 0, "attention_gate_pack: empty shape");
  const int vec_ok = aligned16(x) && aligned16(gate) && aligned16(out) && head_dim % 8 == 0 && x_stride_h % 8 == 0 &&
                     x_stride_t % 8 == 0 && gate_stride_h % 8 == 0 && gate_stride_t % 8 == 0;
  const int64_t total = static_cast<int64_t>(num_tokens) * num_heads * (head_dim / (vec_ok ? 8 : 1));
  const int threads = 256;
  const int64_t want = (total + threads - 1) / threads;
  const unsigned grid = static_cast<unsigned>(want < 1 ? 1 : (want > 148 * 16 ? 148 * 16 : want));
  launch_pdl(chain_overlap(), gate_pack_kernel, dim3(grid), dim3(threads), 0, reinterpret_cast<cudaStream_t>(stream),
             
      static_cast<const __nv_bfloat16*>(x), x_stride_h, x_stride_t, static_cast<const __nv_bfloat16*>(gate),
      gate_stride_h, gate_stride_t, static_cast<__nv_bfloat16*>(out), num_heads, num_tokens, head_dim, vec_ok);
  return check_launch("attention_gate_pack");
}
