// Shared device/host helpers for the sm_100a attention / Gated-DeltaNet kernels.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

namespace b200 {

// ----------------------------------------------------------------------------- model constants
constexpr int PAGE = 16;         // tokens per KV page
constexpr int MAX_SPLITS = 128;  // split-K slots of the reference-compatible split/combine pair
constexpr int HEAD_DIM = 256;    // attention head dim the tensor-core kernels are specialised for
constexpr int GROUP = 4;         // Q heads per KV head
constexpr int GDN_D = 128;       // Gated-DeltaNet key and value dim
constexpr int CHUNK = 64;        // GDN chunk length

// ----------------------------------------------------------------------------- status codes
enum Status : int {
  OK = 0,
  ERR_SHAPE = 1,    // unsupported shape / stride / alignment
  ERR_LAUNCH = 2,   // cudaGetLastError() after the launch
  ERR_RUNTIME = 3,  // other CUDA runtime failure (attribute query, symbol address ...)
  ERR_LIMIT = 4,    // a documented size limit was exceeded
};

void set_error(const char* fmt, ...);
int fail(int code, const char* fmt, ...);
int check_launch(const char* what);
int sm_count();
int* wait_timeout_flag();  // device address of the per-device "a bounded wait ran out" word
bool chain_overlap();      // whether the small decode-step kernels are launched for programmatic dependent launch

#define B200_REQUIRE(cond, ...)                    \
  do {                                             \
    if (!(cond)) return ::b200::fail(::b200::ERR_SHAPE, __VA_ARGS__); \
  } while (0)

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ----------------------------------------------------------------------------- small device helpers
__device__ __forceinline__ float bf16_lo(uint32_t packed) { return __uint_as_float(packed << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t packed) { return __uint_as_float(packed & 0xffff0000u); }

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ float round_bf16(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
// Row count from which the row-wise operators switch to their prompt-sized forms (more bytes in flight per thread;
// below it the one-round-trip forms of the decode step have the shorter latency).
constexpr int GLUE_WIDE_ROWS = 1024;
// SiLU for the prompt-sized element-wise kernels, whose exact exponential and division would cost as many issue slots
// as their memory traffic takes time: fast exponential and reciprocal, a few fp32 ulp before the rounding to bf16.
__device__ __forceinline__ float silu_fast(float a) { return __fdividef(a, 1.0f + __expf(-a)); }

// One RoPE pair with a fixed operation order, so every kernel that rotates produces the same bits.
__device__ __forceinline__ void rope_pair(float a, float b, float sn, float cs, float& first, float& second) {
  first = __fmaf_rn(a, cs, -__fmul_rn(b, sn));
  second = __fmaf_rn(a, sn, __fmul_rn(b, cs));
}

// sigmoid(x) = 0.5 * tanh(x / 2) + 0.5 with the hardware tanh approximation (relative error ~2^-11, far below
// one bf16 ulp): three instructions instead of exp + add + divide.  Used where few warps have a lot of gating to do.
__device__ __forceinline__ float sigmoid_fast(float x) {
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.5f * x));
  return fmaf(t, 0.5f, 0.5f);
}

// 2^x with the hardware approximation (one MUFU instruction; -inf gives 0).
__device__ __forceinline__ float ex2_fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ----------------------------------------------------------------------------- mbarrier + bulk copy (TMA engine)
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: gives up after `limit` polls (each poll may itself block for a hardware-defined time
// slice) and returns false, so a lost copy becomes an error flag instead of a hung GPU.
__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, uint32_t limit = (1u << 22)) {
  // fast path: the copy is usually there within a few polls
  for (int i = 0; i < 64; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
  }
  // slow path: bounded both by poll count and by wall time (about one second)
  const uint64_t t0 = global_timer_ns();
  for (uint32_t i = 0; i < limit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if (global_timer_ns() - t0 > 1000000000ull) return false;
  }
  return false;
}
// 1-D bulk async copy global -> shared, completion counted in bytes on an mbarrier.  dst, src and
// bytes must all be multiples of 16.  No cluster multicast is used anywhere in this library.
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst_smem)),
      "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}
// 1-D bulk async copy shared -> global (same alignment rules), tracked by the issuing thread's bulk group.
__device__ __forceinline__ void bulk_s2g(void* dst_gmem, const void* src_smem, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst_gmem), "r"(smem_u32(src_smem)),
               "r"(bytes)
               : "memory");
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// Wait until the issuing thread's bulk stores have finished READING shared memory (it may then be reused or freed).
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// Barrier among `count` threads (a multiple of 32) that all name the same id (1..15; 0 is __syncthreads).
__device__ __forceinline__ void named_barrier(int id, int count) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ----------------------------------------------------------------------------- programmatic dependent launch
// Overlap flags of the entry points that support it (include/b200_attn.h, B200_OVERLAP_*):
//   START    the kernel is launched with the programmatic-serialization attribute: it may begin while its predecessor
//            in the stream still runs.  What it does before pdl_wait() (barrier set-up, loads of weights) overlaps
//            with the predecessor; pdl_wait() returns once the predecessor has completed and its writes are visible;
//            ALL global writes of the kernel come after it.
//   TRIGGER  the kernel lets its successor begin in the same way (pdl_trigger() at its start).  Only safe when the
//            successor is a kernel that itself waits for its predecessor before it finishes - one of this library's
//            START kernels.  A library kernel launched with the attribute that never waits (an initialisation kernel,
//            say) would complete early, and everything ordered after it would no longer be ordered after this kernel.
//   PREFETCH kernel-specific: also load, before pdl_wait(), state that only an earlier step wrote.
constexpr int OVERLAP_START = 1, OVERLAP_TRIGGER = 2, OVERLAP_PREFETCH = 4;
// NOTE: data written by the predecessor must not be read through a `const __restrict__` pointer: such loads are
// invariant to the compiler, which may hoist them above the wait (seen on the device: a stale projection row).
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
// First statement of the small decode-step kernels (the operators a runner calls one after the other, each a few
// microseconds long): the successor in the stream may be scheduled now, and this kernel touches global memory only after
// its predecessor has completed.  Launched without the attribute (chain_overlap() off) both are no-ops.  The kernels
// that use it take their inputs through plain pointers, never `const __restrict__` (see the note above).
__device__ __forceinline__ void pdl_chain() {
  pdl_trigger();
  pdl_wait();
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(bool early_start, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                              cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = early_start ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// The same with a thread-block cluster of `cluster_x` CTAs along x (grid.x must be a multiple of it).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl_cluster(bool early_start, unsigned cluster_x, void (*kernel)(KArgs...), dim3 grid, dim3 block,
                                      size_t smem, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cluster_x;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = early_start ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// ----------------------------------------------------------------------------- arg-max keys
// (value, index) as one 64-bit key whose unsigned order is "larger value first, then smaller index"; 0 is below every key.
__device__ __forceinline__ unsigned long long argmax_key(float v, uint32_t idx) {
  uint32_t u = __float_as_uint(v);
  u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);  // monotone map of the float order onto unsigned integers
  return (static_cast<unsigned long long>(u) << 32) | (0xffffffffu - idx);
}

// ----------------------------------------------------------------------------- thread-block clusters
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// Barrier over all threads of all CTAs of the cluster (the CTAs of a cluster are co-scheduled, so this cannot wait for
// a CTA that is not running); release / acquire: shared-memory writes before it, local or to a peer, are visible after.
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Address of the same shared-memory location in the CTA of rank `rank` of this cluster.
__device__ __forceinline__ uint32_t cluster_map(uint32_t smem_addr, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(smem_addr), "r"(rank));
  return out;
}
__device__ __forceinline__ void st_cluster_f32x4(uint32_t addr, float a, float b, float c, float d) {
  asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

// ----------------------------------------------------------------------------- warp-level MMA (bf16, fp32 accumulate)
// D[16x8] += A[16x16] * B[16x8]
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
  uint32_t y;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(y) : "r"(x));
  return y;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

}  // namespace b200
