// Paged KV cache writers: single-token append (decode) and packed varlen scatter (prefill).
// Pure byte movement: results are bit-exact with the reference's
// triton_kernels/gqa_attention_decode_paged.py:175-250 (append) and :397-489 (fill).
#include "b200_attn.h"

#include <atomic>
#include "common.cuh"

namespace b200 {

static thread_local char g_error[512] = "";  // per host thread: a caller reads the text of its own failed call
void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}
int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return code;
}
int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(ERR_LAUNCH, "%s: %s", what, cudaGetErrorString(e));
  return OK;
}
// One word per device that kernels set when a bounded wait on a staged copy runs out.
__device__ int g_wait_timeout_flag = 0;
int* wait_timeout_flag() {
  static int* cached[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (!cached[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_wait_timeout_flag) != cudaSuccess) return nullptr;
    cached[dev] = static_cast<int*>(p);
  }
  return cached[dev];
}
// Process-wide switch for the chained launches of the small decode-step kernels (on unless switched off).
static std::atomic<int> g_chain_overlap{1};
bool chain_overlap() { return g_chain_overlap.load(std::memory_order_relaxed) != 0; }

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

// One CTA per (sequence, kv head).  Row = d bf16 elements, moved as 16-byte words.
__global__ void paged_kv_append_kernel(__nv_bfloat16* k_cache, __nv_bfloat16* v_cache,
                                       int64_t kc_p, int64_t kc_h, int64_t kc_s, int64_t vc_p, int64_t vc_h,
                                       int64_t vc_s, const __nv_bfloat16* k_new, int64_t kn_b,
                                       int64_t kn_h, const __nv_bfloat16* v_new, int64_t vn_b,
                                       int64_t vn_h, const int32_t* block_table, int64_t bt_b,
                                       const int64_t* pos, int d, int vec_ok) {
  pdl_chain();
  const int b = blockIdx.x, h = blockIdx.y;
  const int64_t p = pos[b];
  const int64_t lp = p / PAGE, slot = p % PAGE;
  const int64_t phys = static_cast<int64_t>(block_table[b * bt_b + lp]);
  __nv_bfloat16* kd = k_cache + phys * kc_p + h * kc_h + slot * kc_s;
  __nv_bfloat16* vd = v_cache + phys * vc_p + h * vc_h + slot * vc_s;
  const __nv_bfloat16* ks = k_new + b * kn_b + h * kn_h;
  const __nv_bfloat16* vs = v_new + b * vn_b + h * vn_h;
  if (vec_ok) {
    for (int i = threadIdx.x; i < d / 8; i += blockDim.x) {
      reinterpret_cast<uint4*>(kd)[i] = reinterpret_cast<const uint4*>(ks)[i];
      reinterpret_cast<uint4*>(vd)[i] = reinterpret_cast<const uint4*>(vs)[i];
    }
  } else {
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
      kd[i] = ks[i];
      vd[i] = vs[i];
    }
  }
}

// One CTA per (logical page, kv head, sequence); pages past the sequence end exit at once, slots past it
// are neither read nor written.
__global__ void paged_kv_fill_varlen_kernel(__nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache,
                                            int64_t kc_p, int64_t kc_h, int64_t kc_s, int64_t vc_p, int64_t vc_h,
                                            int64_t vc_s, const __nv_bfloat16* __restrict__ k_src, int64_t ks_h,
                                            int64_t ks_t, const __nv_bfloat16* __restrict__ v_src, int64_t vs_h,
                                            int64_t vs_t, const int32_t* __restrict__ block_table, int64_t bt_b,
                                            const int32_t* __restrict__ cu_seqlens, int d, int vec_ok) {
  const int lp = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int start = cu_seqlens[b];
  const int seq_len = cu_seqlens[b + 1] - start;
  if (lp * PAGE >= seq_len) return;
  const int rows = min(PAGE, seq_len - lp * PAGE);
  const int64_t phys = static_cast<int64_t>(block_table[b * bt_b + lp]);
  __nv_bfloat16* kd = k_cache + phys * kc_p + h * kc_h;
  __nv_bfloat16* vd = v_cache + phys * vc_p + h * vc_h;
  const __nv_bfloat16* ks = k_src + h * ks_h + static_cast<int64_t>(start + lp * PAGE) * ks_t;
  const __nv_bfloat16* vs = v_src + h * vs_h + static_cast<int64_t>(start + lp * PAGE) * vs_t;
  if (vec_ok) {
    const int words = d / 8;
    for (int i = threadIdx.x; i < rows * words; i += blockDim.x) {
      const int r = i / words, c = i % words;
      reinterpret_cast<uint4*>(kd + r * kc_s)[c] = reinterpret_cast<const uint4*>(ks + r * ks_t)[c];
      reinterpret_cast<uint4*>(vd + r * vc_s)[c] = reinterpret_cast<const uint4*>(vs + r * vs_t)[c];
    }
  } else {
    for (int i = threadIdx.x; i < rows * d; i += blockDim.x) {
      const int r = i / d, c = i % d;
      kd[r * kc_s + c] = ks[r * ks_t + c];
      vd[r * vc_s + c] = vs[r * vs_t + c];
    }
  }
}

static bool mult8(int64_t x) { return (x & 7) == 0; }

}  // namespace b200

using namespace b200;

extern "C" const char* b200_last_error(void) { return g_error; }
extern "C" int b200_abi_version(void) { return B200_ABI_VERSION; }

extern "C" int b200_set_chain_overlap(int32_t enabled) {
  g_chain_overlap.store(enabled ? 1 : 0);
  return OK;
}

extern "C" int b200_wait_timed_out(void) {
  int* flag = wait_timeout_flag();
  if (!flag) return -1;
  int host = 0;
  if (cudaMemcpy(&host, flag, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  if (host) cudaMemset(flag, 0, sizeof(int));
  return host;
}

extern "C" int b200_paged_kv_append(void* k_cache, void* v_cache, int64_t kc_stride_p, int64_t kc_stride_h,
                                    int64_t kc_stride_s, int64_t vc_stride_p, int64_t vc_stride_h,
                                    int64_t vc_stride_s, const void* k_new, int64_t kn_stride_b, int64_t kn_stride_h,
                                    const void* v_new, int64_t vn_stride_b, int64_t vn_stride_h,
                                    const int32_t* block_table, int64_t bt_stride_b, const int64_t* pos,
                                    int32_t batch, int32_t num_kv_heads, int32_t head_dim, b200_stream_t stream) {
  B200_REQUIRE(batch > 0 && num_kv_heads > 0 && head_dim > 0, "paged_kv_append: empty shape");
  B200_REQUIRE(num_kv_heads <= 65535, "paged_kv_append: too many heads");
  const int vec_ok = aligned16(k_cache) && aligned16(v_cache) && aligned16(k_new) && aligned16(v_new) &&
                     mult8(head_dim) && mult8(kc_stride_p) && mult8(kc_stride_h) && mult8(kc_stride_s) &&
                     mult8(vc_stride_p) && mult8(vc_stride_h) && mult8(vc_stride_s) && mult8(kn_stride_b) &&
                     mult8(kn_stride_h) && mult8(vn_stride_b) && mult8(vn_stride_h);
  launch_pdl(chain_overlap(), paged_kv_append_kernel, dim3(batch, num_kv_heads), dim3(32), 0, reinterpret_cast<cudaStream_t>(stream),
             
      static_cast<__nv_bfloat16*>(k_cache), static_cast<__nv_bfloat16*>(v_cache), kc_stride_p, kc_stride_h,
      kc_stride_s, vc_stride_p, vc_stride_h, vc_stride_s, static_cast<const __nv_bfloat16*>(k_new), kn_stride_b,
      kn_stride_h, static_cast<const __nv_bfloat16*>(v_new), vn_stride_b, vn_stride_h, block_table, bt_stride_b, pos,
      head_dim, vec_ok);
  return check_launch("paged_kv_append");
}

extern "C" int b200_paged_kv_fill_varlen(void* k_cache, void* v_cache, int64_t kc_stride_p, int64_t kc_stride_h,
                                         int64_t kc_stride_s, int64_t vc_stride_p, int64_t vc_stride_h,
                                         int64_t vc_stride_s, const void* k_packed, int64_t kp_stride_h,
                                         int64_t kp_stride_t, const void* v_packed, int64_t vp_stride_h,
                                         int64_t vp_stride_t, const int32_t* block_table, int64_t bt_stride_b,
                                         const int32_t* cu_seqlens, int32_t batch, int32_t num_kv_heads,
                                         int32_t head_dim, int32_t max_seqlen, b200_stream_t stream) {
  B200_REQUIRE(batch > 0 && num_kv_heads > 0 && head_dim > 0, "paged_kv_fill_varlen: empty shape");
  B200_REQUIRE(batch <= 65535 && num_kv_heads <= 65535, "paged_kv_fill_varlen: grid too large");
  if (max_seqlen <= 0) return OK;
  const int vec_ok = aligned16(k_cache) && aligned16(v_cache) && aligned16(k_packed) && aligned16(v_packed) &&
                     mult8(head_dim) && mult8(kc_stride_p) && mult8(kc_stride_h) && mult8(kc_stride_s) &&
                     mult8(vc_stride_p) && mult8(vc_stride_h) && mult8(vc_stride_s) && mult8(kp_stride_h) &&
                     mult8(kp_stride_t) && mult8(vp_stride_h) && mult8(vp_stride_t);
  const int pages = (max_seqlen + PAGE - 1) / PAGE;
  paged_kv_fill_varlen_kernel<<<dim3(pages, num_kv_heads, batch), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16*>(k_cache), static_cast<__nv_bfloat16*>(v_cache), kc_stride_p, kc_stride_h,
      kc_stride_s, vc_stride_p, vc_stride_h, vc_stride_s, static_cast<const __nv_bfloat16*>(k_packed), kp_stride_h,
      kp_stride_t, static_cast<const __nv_bfloat16*>(v_packed), vp_stride_h, vp_stride_t, block_table, bt_stride_b,
      cu_seqlens, head_dim, vec_ok);
  return check_launch("paged_kv_fill_varlen");
}
