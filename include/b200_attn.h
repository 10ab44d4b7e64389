/*
 * b200_attn.h -- C ABI of libb200attn.so: hand-written sm_100a CUDA kernels for the attention /
 * Gated-DeltaNet hot path of a Qwen3.5-style decoder.
 *
 * Every entry point replaces one operator of the reference engine (cited as file:line inside the
 * reference project) and keeps its argument meaning.  Conventions:
 *   - All pointers are DEVICE pointers unless a comment says "host".  bf16 tensors are passed as
 *     `void*`, fp32 as `float*`, page tables / cu_seqlens as `int32_t*`, positions as `int64_t*`.
 *   - Strides are in ELEMENTS.  The innermost dimension of every tensor must have stride 1.
 *   - `stream` is the cudaStream_t to launch on (0 = legacy default stream).
 *   - Return value: 0 = kernel launched; non-zero = nothing was launched, b200_last_error() says why.
 *   - The entry points that replace a reference operator, and the two fused attention steps, neither synchronise,
 *     nor allocate device memory, nor read device data on the host, so they may be captured into a CUDA graph
 *     (exceptions are marked "host-synchronous").
 *   - Kernels do no bounds checks on page ids or positions: sizing the page table is the caller's job,
 *     exactly as in the reference (triton_kernels/gqa_attention_decode_paged.py:225-226).
 */
#ifndef B200_ATTN_H_
#define B200_ATTN_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200_ABI_VERSION 1

/* Model constants the tensor-core kernels are specialised for (other values are rejected). */
#define B200_PAGE_SIZE 16   /* triton_kernels/gqa_attention_decode_paged.py:91  PAGE_SIZE  */
#define B200_MAX_SPLITS 128 /* triton_kernels/gqa_attention_decode_paged.py:95  MAX_SPLITS */
#define B200_HEAD_DIM 256
#define B200_GROUP 4
#define B200_GDN_DIM 128
#define B200_GDN_CHUNK 64

typedef void* b200_stream_t; /* cudaStream_t */

/* ------------------------------------------------------------------------------------------ utilities */
const char* b200_last_error(void); /* host string describing the last non-zero return */
int b200_abi_version(void);
/* host-synchronous: 1 if a kernel on the current device gave up a bounded wait on a staged copy since the
 * last call (the flag is cleared), 0 if not, -1 on a runtime error.  For tests and debugging. */
int b200_wait_timed_out(void);

/* The small operators of a decode step (partial_rope, attention_gate_pack, paged_kv_append, the split / combine pair,
 * gdn_recurrent_decode, the decode conv, the GDN norms and gates, residual_add, embedding_gather) are each a few
 * microseconds long and are called one after the other; they are launched for programmatic dependent launch: every such
 * kernel lets its successor in the stream be scheduled at once and itself touches global memory only after its
 * predecessor has completed, so the launch latencies overlap instead of adding up (a kernel of another library in
 * between is unaffected: it starts when its predecessor has finished, as always).  b200_set_chain_overlap(0) launches
 * them plainly again, process-wide (for comparisons, or under tools that do not model such launches).  No counterpart
 * in the reference. */
int b200_set_chain_overlap(int32_t enabled);

/* Diagnostic: one CTA multiplies two bf16 tiles loaded by tensor-map TMA with tcgen05.mma (accumulator in tensor
 * memory) and writes fp32 C.  mode 0: C[128x64] = A[128x256] . B[64x256]^T;  mode 1: C[128x256] = A[128x64] . B[64x256];
 * mode 2: as mode 1 with A handed to the MMA through tensor memory instead of shared memory.
 * All matrices row-major and contiguous.  No counterpart in the reference; it validates the sm_100a building blocks
 * the prefill kernels use. */
int b200_selftest_umma(int32_t mode, const void* a, const void* b, float* c, b200_stream_t stream);
/* Diagnostic: one warp waits, with a small poll limit, on a staged-copy barrier that nothing will ever complete.  The
 * wait gives up, the kernel sets the flag that b200_wait_timed_out() reports, leaves *sentinel (device int32) as it was
 * and returns; nothing faults or hangs.  It exercises the give-up path that every kernel of this library takes when a
 * copy it waits for does not arrive.  No counterpart in the reference. */
int b200_selftest_wait_timeout(int32_t* sentinel, b200_stream_t stream);

/* ------------------------------------------------------------------------------------------ paged KV cache */
/* cache[block_table[b, pos[b]/16], h, pos[b]%16, :] = new[b, h, :] for K and V.
 * Replaces wy_lib::paged_kv_append, triton_kernels/gqa_attention_decode_paged.py:254-305 (kernel :175-250).
 * caches [num_pages, H_kv, 16, D] bf16; k_new/v_new [B, H_kv, D] bf16; block_table [B, max_pages]; pos [B]. */
int b200_paged_kv_append(void* k_cache, void* v_cache, int64_t kc_stride_p, int64_t kc_stride_h, int64_t kc_stride_s,
                         int64_t vc_stride_p, int64_t vc_stride_h, int64_t vc_stride_s, const void* k_new,
                         int64_t kn_stride_b, int64_t kn_stride_h, const void* v_new, int64_t vn_stride_b,
                         int64_t vn_stride_h, const int32_t* block_table, int64_t bt_stride_b, const int64_t* pos,
                         int32_t batch, int32_t num_kv_heads, int32_t head_dim, b200_stream_t stream);

/* Scatter packed K/V [H_kv, T, D] (any h/t strides) into each sequence's pages; slots past a sequence's end
 * keep their bytes.  max_seqlen (host) only sizes the grid.
 * Replaces wy_lib::paged_kv_fill_varlen, triton_kernels/gqa_attention_decode_paged.py:492-561 (kernel :397-489). */
int b200_paged_kv_fill_varlen(void* k_cache, void* v_cache, int64_t kc_stride_p, int64_t kc_stride_h,
                              int64_t kc_stride_s, int64_t vc_stride_p, int64_t vc_stride_h, int64_t vc_stride_s,
                              const void* k_packed, int64_t kp_stride_h, int64_t kp_stride_t, const void* v_packed,
                              int64_t vp_stride_h, int64_t vp_stride_t, const int32_t* block_table,
                              int64_t bt_stride_b, const int32_t* cu_seqlens, int32_t batch, int32_t num_kv_heads,
                              int32_t head_dim, int32_t max_seqlen, b200_stream_t stream);

/* ------------------------------------------------------------------------------------------ paged decode attention */
/* Split-K partial attention with the reference's page partition; writes all 128 (m, l, acc) partials.
 * q [B, H_q, 256] bf16; m_partial/l_partial [B, H_q, 128] fp32, acc_partial [B, H_q, 128, 256] fp32, contiguous.
 * Replaces wy_lib::paged_gqa_attention_decode_split, triton_kernels/gqa_attention_decode_paged.py:822-891
 * (kernel :622-733). */
int b200_paged_decode_split(const void* q, int64_t q_stride_b, int64_t q_stride_h, const void* k_cache,
                            const void* v_cache, int64_t kc_stride_p, int64_t kc_stride_h, int64_t kc_stride_s,
                            int64_t vc_stride_p, int64_t vc_stride_h, int64_t vc_stride_s, const int32_t* block_table,
                            int64_t bt_stride_b, float* m_partial, float* l_partial, float* acc_partial,
                            const int64_t* pos, int32_t batch, int32_t num_q_heads, int32_t num_kv_heads,
                            int32_t head_dim, b200_stream_t stream);

/* Merge the active partials into out [B, H_q, 256] bf16 (contiguous).
 * Replaces wy_lib::paged_gqa_attention_decode_combine, triton_kernels/gqa_attention_decode_paged.py:901-939
 * (kernel :745-817). */
int b200_paged_decode_combine(const float* m_partial, const float* l_partial, const float* acc_partial,
                              const int64_t* pos, void* out, int32_t batch, int32_t num_q_heads, int32_t head_dim,
                              b200_stream_t stream);

/* Fused decode attention layer core: partial RoPE on q and k_new at position pos[b], append of the rotated
 * k_new and of v_new to the paged cache, attention over the pos[b]+1 cached tokens, sigmoid output gate.
 * One launch replaces the chain partial_rope x2 -> paged_kv_append -> split -> combine -> attention_gate_pack of
 * engine/runner.py:482-517 (call_paged_gqa_attention_decode_triton, gqa_attention_decode_paged.py:963-994).
 * q [B,H_q,256], k_new/v_new [B,H_kv,256], gate [B, H_q*256] (row stride gate_stride_b), out [B, H_q*256] bf16
 * contiguous; inv_freq [rotary_dim/2] fp32; rotary_dim is 64 (the model's) or 0 = no rotation; gate may be NULL:
 * out is then bf16(acc / l), what the reference's combine kernel returns (with rotary_dim 0 the call is
 * call_paged_gqa_attention_decode_triton itself: append + attention, one launch instead of three).  The pools must be
 * the dense [num_pages, H_kv, 16, 256] layout (pages are fetched by tensor-map TMA, one 8 KiB box per page and head).
 * workspace: b200_fused_decode_workspace_bytes() bytes of device memory, 256-byte aligned, zero-filled ONCE by
 * the caller before the first use (the kernel leaves it zeroed again); calls sharing a workspace must not
 * overlap on the device. */
int64_t b200_fused_decode_workspace_bytes(void);
int b200_fused_decode_attention(const void* q, int64_t q_stride_b, int64_t q_stride_h, const void* k_new,
                                int64_t kn_stride_b, int64_t kn_stride_h, const void* v_new, int64_t vn_stride_b,
                                int64_t vn_stride_h, const void* gate, int64_t gate_stride_b, void* k_cache,
                                void* v_cache, int64_t kc_stride_p, int64_t kc_stride_h, int64_t kc_stride_s,
                                int64_t vc_stride_p, int64_t vc_stride_h, int64_t vc_stride_s, int64_t num_pages,
                                const int32_t* block_table, int64_t bt_stride_b, const int64_t* pos,
                                const float* inv_freq, int32_t rotary_dim, void* out, void* workspace, int32_t batch,
                                int32_t num_q_heads, int32_t num_kv_heads, int32_t head_dim, b200_stream_t stream);

/* b200_fused_decode_attention with two optional extensions.
 * q_norm_weight / k_norm_weight (bf16 [head_dim], or NULL): the per-head Qwen RMSNorm x * rsqrt(mean(x^2) + eps) *
 *   (1 + weight) of q and k_new (triton_kernels/qwen_rmsnorm.py:70-73 as applied at engine/runner.py:476-489) is computed
 *   inside the kernel, rounded to bf16 like the reference's q_norm / k_norm output, before the RoPE; q and k_new are
 *   then the raw projections.  Same bytes as b200_add_rmsnorm followed by the plain call.
 * overlap (B200_OVERLAP_*, defined below): START lets the kernel begin while the kernel in front of it still runs;
 *   PREFETCH additionally lets it compute the position prefix, gather page ids and request its first K/V pages before
 *   that kernel has finished - pass it only when that kernel writes neither pos, the block table nor the caches (in a
 *   layer stack it is the q/k/v/gate projection).  q, k_new, v_new and gate are always read after it.
 * partition: how the KV pages are cut over the CTAs.  0 = the kernel chooses per launch from the lengths in pos[];
 *   1 = always equal ranges of pages per CTA (segments cut at range boundaries are merged through the workspace);
 *   2 = always one whole (sequence, kv head) segment per CTA (needs batch * num_kv_heads <= the number of SMs, else the
 *   call is refused); 3 = always one segment per thread-block cluster, whose CTAs share the segment's pages and merge
 *   through distributed shared memory (needs batch * num_kv_heads <= 64, else refused).  The result is the same up to
 *   fp32 summation order; 1, 2 and 3 exist so that tests and tuning can pin each form. */
int b200_fused_decode_attention_ex(const void* q, int64_t q_stride_b, int64_t q_stride_h, const void* k_new,
                                   int64_t kn_stride_b, int64_t kn_stride_h, const void* v_new, int64_t vn_stride_b,
                                   int64_t vn_stride_h, const void* gate, int64_t gate_stride_b, void* k_cache,
                                   void* v_cache, int64_t kc_stride_p, int64_t kc_stride_h, int64_t kc_stride_s,
                                   int64_t vc_stride_p, int64_t vc_stride_h, int64_t vc_stride_s, int64_t num_pages,
                                   const int32_t* block_table, int64_t bt_stride_b, const int64_t* pos,
                                   const float* inv_freq, int32_t rotary_dim, void* out, void* workspace, int32_t batch,
                                   int32_t num_q_heads, int32_t num_kv_heads, int32_t head_dim,
                                   const void* q_norm_weight, const void* k_norm_weight, float eps, int32_t overlap,
                                   int32_t partition, b200_stream_t stream);

/* The same fused decode step for callers that cannot allocate device memory (a host that owns the whole GPU and
 * forbids cudaMalloc after start-up, a plugin inside another process, code running under stream capture).  This
 * entry point has NO counterpart in the reference.  Arguments are those of b200_fused_decode_attention without
 * `workspace`: the workspace is a fixed ~2 MB array inside the library's device image (present on every GPU that
 * loads the library, until the process exits).  Nothing is allocated, here or in anything it calls.
 *   - Limits: batch <= 512 and batch * num_kv_heads <= 2048; larger calls return non-zero and launch nothing.
 *   - The first call on a device also resolves the array's device address: make it before any stream capture.
 *   - All calls on a device share the array; it is re-initialised on `stream` at the start of each call, so calls
 *     that overlap on the GPU race and must be serialised by the caller. */
int b200_fused_decode_attention_static(const void* q, int64_t q_stride_b, int64_t q_stride_h, const void* k_new,
                                       int64_t kn_stride_b, int64_t kn_stride_h, const void* v_new,
                                       int64_t vn_stride_b, int64_t vn_stride_h, const void* gate,
                                       int64_t gate_stride_b, void* k_cache, void* v_cache, int64_t kc_stride_p,
                                       int64_t kc_stride_h, int64_t kc_stride_s, int64_t vc_stride_p,
                                       int64_t vc_stride_h, int64_t vc_stride_s, int64_t num_pages,
                                       const int32_t* block_table, int64_t bt_stride_b, const int64_t* pos,
                                       const float* inv_freq,
                                       int32_t rotary_dim, void* out, int32_t batch, int32_t num_q_heads,
                                       int32_t num_kv_heads, int32_t head_dim, b200_stream_t stream);

/* ------------------------------------------------------------------------------------------ varlen causal prefill attention */
/* Block-diagonal causal GQA over a packed batch: q [T,H_q,256], k/v [T,H_kv,256] bf16 (any t/h strides),
 * cu_seqlens [B+1] int32, out [T,H_q,256] bf16.  total_tokens = T bounds the TMA tensor maps; max_seqlen (host) only
 * sizes the grid.  Runs on tcgen05 tensor cores with accumulators in tensor memory.
 * Replaces wy_lib::gqa_attention_varlen_causal, triton_kernels/gqa_attention_varlen_causal.py:214-278
 * (kernel :99-210). */
int b200_gqa_varlen_causal(const void* q, int64_t q_stride_t, int64_t q_stride_h, const void* k, int64_t k_stride_t,
                           int64_t k_stride_h, const void* v, int64_t v_stride_t, int64_t v_stride_h, void* out,
                           int64_t out_stride_t, int64_t out_stride_h, const int32_t* cu_seqlens, int32_t batch,
                           int32_t total_tokens, int32_t max_seqlen, int32_t num_q_heads, int32_t num_kv_heads,
                           int32_t head_dim, b200_stream_t stream);

/* Fused prefill attention layer core in two launches: (1) partial RoPE on k at position_ids[t], scatter of the
 * rotated k and of v into the paged cache, and a packed copy of the rotated k into k_rot_scratch; (2) partial RoPE on
 * q in shared memory, causal attention on the tensor cores (tcgen05/TMEM), sigmoid output gate.  Replaces the chain
 * partial_rope x2 -> gqa_attention_varlen_causal -> attention_gate_pack -> paged_kv_fill_varlen of
 * engine/runner.py:339-384.
 * q [T,H_q,256], k/v [T,H_kv,256] are the post-norm PRE-RoPE projections; gate [T, H_q*256] (row stride
 * gate_stride_t); position_ids [T] int32/int64; k_rot_scratch: T*H_kv*256 bf16 of caller-owned device memory
 * (contents undefined afterwards); out [T, H_q*256] bf16 contiguous; rotary_dim must be 64. */
int b200_fused_prefill_attention(const void* q, int64_t q_stride_t, int64_t q_stride_h, const void* k,
                                 int64_t k_stride_t, int64_t k_stride_h, const void* v, int64_t v_stride_t,
                                 int64_t v_stride_h, const void* gate, int64_t gate_stride_t, void* k_cache,
                                 void* v_cache, int64_t kc_stride_p, int64_t kc_stride_h, int64_t kc_stride_s,
                                 int64_t vc_stride_p, int64_t vc_stride_h, int64_t vc_stride_s,
                                 const int32_t* block_table, int64_t bt_stride_b, const int32_t* cu_seqlens,
                                 const void* position_ids, int32_t ids_are_int64, const float* inv_freq,
                                 int32_t rotary_dim, void* k_rot_scratch, void* out, int32_t batch,
                                 int32_t total_tokens, int32_t max_seqlen, int32_t num_q_heads, int32_t num_kv_heads,
                                 int32_t head_dim, b200_stream_t stream);

/* ------------------------------------------------------------------------------------------ rope / gate */
/* Half-split rotation of the first rotary_dim dims of x [B,H,T,D] bf16 (dims >= rotary_dim copied).
 * position_ids [B,T] int32 or int64.  Replaces wy_lib::partial_rope, triton_kernels/partial_rope.py:145-198
 * (kernel :27-132). */
int b200_partial_rope(const void* x, int64_t x_stride_b, int64_t x_stride_h, int64_t x_stride_t, void* out,
                      int64_t out_stride_b, int64_t out_stride_h, int64_t out_stride_t, const void* position_ids,
                      int32_t ids_are_int64, int64_t ids_stride_b, int64_t ids_stride_t, const float* inv_freq,
                      int32_t batch, int32_t num_heads, int32_t num_tokens, int32_t head_dim, int32_t rotary_dim,
                      b200_stream_t stream);

/* out[t, h*D + d] = bf16(x[h,t,d] * sigmoid(gate[h,t,d])); x, gate are [1,H,T,D] views, out [T, H*D] contiguous.
 * Replaces wy_lib::attention_gate_pack, triton_kernels/attention_gate_pack.py:77-126 (kernel :15-64). */
int b200_attention_gate_pack(const void* x, int64_t x_stride_h, int64_t x_stride_t, const void* gate,
                             int64_t gate_stride_h, int64_t gate_stride_t, void* out, int32_t num_heads,
                             int32_t num_tokens, int32_t head_dim, b200_stream_t stream);

/* ------------------------------------------------------------------------------------------ Gated DeltaNet */
/* One delta-rule step per sequence; state [B,H,128,128] fp32 updated in place (inner two dims contiguous).
 * q,k [B,H,128] bf16, v [B,H,128] bf16 (any b/h strides), beta,g [B,H] fp32, out [B,H,128] bf16.
 * Replaces wy_lib::gdn_recurrent_decode, triton_kernels/gdn_recurrent_prefill.py:1185-1259 (kernel :145-246). */
int b200_gdn_recurrent_decode(const void* q, int64_t q_stride_b, int64_t q_stride_h, const void* k,
                              int64_t k_stride_b, int64_t k_stride_h, const void* v, int64_t v_stride_b,
                              int64_t v_stride_h, const float* beta, int64_t beta_stride_b, int64_t beta_stride_h,
                              const float* g, int64_t g_stride_b, int64_t g_stride_h, float* state,
                              int64_t state_stride_b, int64_t state_stride_h, void* out, int64_t out_stride_b,
                              int64_t out_stride_h, int32_t batch, int32_t num_heads, int32_t key_dim,
                              int32_t value_dim, b200_stream_t stream);

/* Diagnostic: pins the kernel form b200_gdn_recurrent_decode takes, process-wide (0 = chosen from the sizes, the
 * default; 1 = one CTA per head with the state in registers; 2 = one warp per 32 value columns; 3 = persistent CTAs,
 * eight per SM, that stream [128 x 16] boxes of the state through a shared-memory ring of three with tensor-map TMA
 * copies issued by a copy warp).  A form whose layout rules do not hold for a call falls back to 1.  The same switch
 * pins b200_gdn_decode_fused: 1 = a head's state in registers, 3 = whole heads streamed as [128 x 32] boxes through a
 * ring of three, four CTAs per SM (its default from more heads than two register-resident CTAs per SM hold).  For tests
 * and tuning: every form computes the same step (fp32 summation order differs).  No counterpart in the reference. */
int b200_gdn_recurrent_decode_form(int32_t form);

/* Token-serial recurrence over a packed buffer, zero state at every cu_seqlens[b]; cu_seqlens may be NULL
 * (one sequence of total_tokens).  state [batch,H,128,128] fp32 contiguous (written), out [T,H,128] bf16.
 * Replaces wy_lib::gdn_recurrent_prefill_sequential, triton_kernels/gdn_recurrent_prefill.py:1050-1145
 * (kernel :47-143). */
int b200_gdn_recurrent_prefill_sequential(const void* q, int64_t q_stride_t, int64_t q_stride_h, const void* k,
                                          int64_t k_stride_t, int64_t k_stride_h, const void* v, int64_t v_stride_t,
                                          int64_t v_stride_h, const float* beta, int64_t beta_stride_t,
                                          int64_t beta_stride_h, const float* g, int64_t g_stride_t,
                                          int64_t g_stride_h, const int32_t* cu_seqlens, int32_t batch,
                                          int32_t total_tokens, float* state, void* out, int64_t out_stride_t,
                                          int64_t out_stride_h, int32_t num_heads, int32_t key_dim, int32_t value_dim,
                                          b200_stream_t stream);

/* Chunk-64 form of the recurrence for ONE sequence of token_num tokens, as the reference's three operators with
 * their fp32 intermediates (N = cdiv(token_num, 64); every output is contiguous):
 *   prepare_wy: w [N,H,64,128], u_base [N,H,64,128], g_cumsum [N,H,64]
 *               replaces wy_lib::gdn_chunk_prepare_wy, triton_kernels/gdn_recurrent_prefill.py:703-784 (kernel :248-396)
 *   state:      delta [N,H,64,128], chunk_state [N,H,128,128] (state ENTERING each chunk), final_state [H,128,128]
 *               replaces wy_lib::gdn_chunk_state, triton_kernels/gdn_recurrent_prefill.py:825-909 (kernel :404-537)
 *   output:     out [T,H,128] bf16
 *               replaces wy_lib::gdn_chunk_output, triton_kernels/gdn_recurrent_prefill.py:935-1006 (kernel :563-690) */
int b200_gdn_chunk_prepare_wy(const void* k, int64_t k_stride_t, int64_t k_stride_h, const void* v, int64_t v_stride_t,
                              int64_t v_stride_h, const float* beta, int64_t beta_stride_t, int64_t beta_stride_h,
                              const float* g, int64_t g_stride_t, int64_t g_stride_h, float* w, float* u_base,
                              float* g_cumsum, int32_t token_num, int32_t num_heads, int32_t key_dim,
                              int32_t value_dim, b200_stream_t stream);
int b200_gdn_chunk_state(const void* k, int64_t k_stride_t, int64_t k_stride_h, const float* w, const float* u_base,
                         const float* g_cumsum, float* delta, float* chunk_state, float* final_state,
                         int32_t token_num, int32_t num_heads, int32_t key_dim, int32_t value_dim,
                         b200_stream_t stream);
int b200_gdn_chunk_output(const void* q, int64_t q_stride_t, int64_t q_stride_h, const void* k, int64_t k_stride_t,
                          int64_t k_stride_h, const float* delta, const float* g_cumsum, const float* chunk_state,
                          void* out, int64_t out_stride_t, int64_t out_stride_h, int32_t token_num, int32_t num_heads,
                          int32_t key_dim, int32_t value_dim, b200_stream_t stream);

/* Chunk-64 prefill over a PACKED batch: the three stages above with the chunk grid restarting at every
 * cu_seqlens[b] and a zero state at each sequence start; out [T,H,128] bf16, state [batch,H,128,128] fp32 (written).
 * The reference's chunk path is single-sequence (engine/runner.py:263-267, README-EN.md:306-308); this packed form
 * equals wy_lib::gdn_recurrent_prefill_sequential(..., cu_seqlens) up to fp32 rounding.  `workspace` is
 * b200_gdn_chunked_prefill_packed_workspace_bytes(batch, total_tokens, num_heads) bytes of caller-owned device
 * memory, 16-byte aligned (contents undefined afterwards); max_seqlen (host) only sizes the grid. */
int64_t b200_gdn_chunked_prefill_packed_workspace_bytes(int32_t batch, int32_t total_tokens, int32_t num_heads);
int b200_gdn_chunked_prefill_packed(const void* q, int64_t q_stride_t, int64_t q_stride_h, const void* k,
                                    int64_t k_stride_t, int64_t k_stride_h, const void* v, int64_t v_stride_t,
                                    int64_t v_stride_h, const float* beta, int64_t beta_stride_t,
                                    int64_t beta_stride_h, const float* g, int64_t g_stride_t, int64_t g_stride_h,
                                    const int32_t* cu_seqlens, int32_t batch, int32_t total_tokens, int32_t max_seqlen,
                                    void* workspace, float* state, void* out, int64_t out_stride_t,
                                    int64_t out_stride_h, int32_t num_heads, int32_t key_dim, int32_t value_dim,
                                    b200_stream_t stream);

/* The same packed chunk-64 prefill as ONE kernel on the tcgen05 tensor cores: one CTA per (sequence, head) keeps the
 * state in tensor memory and walks the chunks; Q/K/V chunks arrive by tensor-map TMA, no workspace, no max_seqlen.
 * q, k, v must be 16-byte aligned with token and head strides that are multiples of 8 elements.  No reference
 * counterpart as a single call (it fuses triton_kernels/gdn_recurrent_prefill.py:703-784, :825-909, :935-1006 for a
 * packed batch); results equal wy_lib::gdn_recurrent_prefill_sequential(..., cu_seqlens) within the reference's
 * chunked-vs-sequential bars (out 1e-2, state 5e-4, gdn_recurrent_prefill.py:1520-1526). */
int b200_gdn_chunked_prefill_fused(const void* q, int64_t q_stride_t, int64_t q_stride_h, const void* k,
                                   int64_t k_stride_t, int64_t k_stride_h, const void* v, int64_t v_stride_t,
                                   int64_t v_stride_h, const float* beta, int64_t beta_stride_t,
                                   int64_t beta_stride_h, const float* g, int64_t g_stride_t, int64_t g_stride_h,
                                   const int32_t* cu_seqlens, int32_t batch, int32_t total_tokens, float* state,
                                   void* out, int64_t out_stride_t, int64_t out_stride_h, int32_t num_heads,
                                   int32_t key_dim, int32_t value_dim, b200_stream_t stream);

/* ------------------------------------------------------------------------------------------------------------------
 * Row-wise layer operators around the projections (one launch each).  bf16 tensors, fp32 math, one rounding at the
 * reference's rounding points.
 *
 * b200_add_rmsnorm: norm_out[r,:] = s * rsqrt(mean(s^2) + eps) * (1 + weight), s = x[r,:] (+ residual[r,:], rounded
 * to bf16 first and also written to sum_out when that is non-NULL).  Row r of x lives at
 * x + (r / inner_count) * x_stride_outer + (r % inner_count) * x_stride_inner (so a [n, H, D] column view of a fused
 * projection works); residual rows are residual_stride apart; sum_out and norm_out are contiguous [rows, dim].
 * dim must be a multiple of 256, at most 8192.  Replaces triton_kernels/qwen_rmsnorm.py:98-146 (and
 * triton_kernels/residual_add.py in front of it).
 * b200_swiglu: out[r, c] = silu(gate_up[r, c]) * gate_up[r, intermediate + c].  Replaces triton_kernels/swiglu.py.
 * b200_gdn_decode_prep: one decode token per sequence of a Gated-DeltaNet layer: shifts conv_state [B,4,3*H*128]
 * left and appends qkv (triton_kernels/depthwise_causal_conv4_decode.py), y = silu(sum_r weight4[r,c] state[r,c])
 * rounded to bf16, then q_out = l2norm(y_q) * 128^-0.5, k_out = l2norm(y_k), v_out = y_v as contiguous [B,H,128] and
 * beta = sigmoid(b), g = -exp(a_log) * softplus(a + dt_bias) as fp32 [B,H] (triton_kernels/gdn_qk_norm_gates.py:68-89).
 * b200_gdn_gated_rmsnorm: out[r,:] = x[r,:] * rsqrt(mean(x^2) + 1e-6) * weight * silu(z[r,:]) for rows r = (n, head);
 * x and out contiguous [rows, 128], z row (n, head) at z + n * z_stride + head * 128
 * (triton_kernels/gdn_gated_rmsnorm.py:95-140). */
/* Overlap flags (programmatic dependent launch) of b200_(norm_)skinny_gemm, b200_add_rmsnorm, b200_swiglu and
 * b200_gdn_decode_fused; 0 = plain stream order.
 *   START    the kernel may begin while the kernel in front of it in the stream still runs; it reads that kernel's
 *            output, and writes anything, only after that kernel has completed.
 *   TRIGGER  the kernel lets the NEXT kernel in the stream begin early in the same way.  Pass it only when that next
 *            kernel is one of these four launched with START: a kernel that does not itself wait for its predecessor
 *            before finishing (some library initialisation kernels) would break the ordering of everything after it.
 *   PREFETCH b200_gdn_decode_fused only, see there. */
#define B200_OVERLAP_START 1
#define B200_OVERLAP_TRIGGER 2
#define B200_OVERLAP_PREFETCH 4

/* The whole Gated-DeltaNet mixer of ONE decode token per sequence between its two projections, one launch:
 * b200_gdn_decode_prep -> b200_gdn_recurrent_decode -> b200_gdn_gated_rmsnorm with nothing written in between.
 * fused: one row per sequence of the input projection, [q | k | v | z | a | b] = [3*H*128 | H*128 | H | H] bf16, rows
 * fused_stride elements apart; conv_state [B,4,3*H*128] bf16 and state [B,H,128,128] fp32 are updated in place;
 * weight4 [4,3*H*128] bf16, a_log [H] fp32, dt_bias [H] bf16, norm_weight [128] fp32; out [B, H*128] bf16 contiguous.
 * Replaces the operator chain of engine/runner.py:431-441.  `overlap`: B200_OVERLAP_* flags (below); PREFETCH lets the
 * kernel load conv_state and state before the kernel in front of it has finished - pass it only when that kernel does
 * not write them (in a layer stack it is the input projection).  Large batches stream the state through a TMA ring
 * (see b200_gdn_recurrent_decode_form); a bounded wait of that form that runs out leaves the head's state and output
 * untouched and sets b200_wait_timed_out(). */
int b200_gdn_decode_fused(const void* fused, int64_t fused_stride, void* conv_state, const void* weight4,
                          const float* a_log, const void* dt_bias, const float* norm_weight, float* state, void* out,
                          int32_t batch, int32_t num_heads, int32_t head_dim, int32_t overlap, b200_stream_t stream);
/* Y[M,N] = X[M,K] . W[N,K]^T for decode batches (M <= 32), bf16 in/out, fp32 accumulation: W is streamed once by
 * tensor-map TMA, X staged in shared memory.  N a multiple of 8, K a multiple of 128.  K <= 1280: every warp owns 16
 * outputs and all of K.  K > 1280 (up to 16384; the projections back to the hidden size): a CTA owns 16 outputs, its
 * warps split K and X is staged in ceil(K/1024) equal chunks, which must consist of whole 128-k tiles (2048 and 3584
 * do).  x / y rows x_stride / y_stride elements apart (multiples of 8), weight contiguous [N,K]; all 16-byte aligned.  With
 * B200_OVERLAP_START the weight tiles are requested before the preceding kernel in the stream has finished, so
 * `weight` must not be that kernel's output (x may be).
 * Replaces triton_kernels/gemm_2d.py for the decode-step projections of the hidden state. */
int b200_skinny_gemm(const void* x, int64_t x_stride, const void* weight, void* y, int64_t y_stride, int32_t m,
                     int32_t n, int32_t k, int32_t overlap, b200_stream_t stream);
/* The gate/up projection of the MLP with its activation folded into the epilogue (one launch instead of two):
 *   weight = [gate rows | up rows] [2*intermediate, K];  y[:, j] = silu(bf16(x . gate_j)) * bf16(x . up_j)
 * (triton_kernels/gemm_2d.py on the fused gate/up weight followed by triton_kernels/swiglu.py).  y is
 * [M, intermediate]; intermediate a multiple of 8; other shapes, alignment and overlap flags as b200_skinny_gemm. */
int b200_skinny_gemm_swiglu(const void* x, int64_t x_stride, const void* weight, void* y, int64_t y_stride, int32_t m,
                            int32_t intermediate, int32_t k, int32_t overlap, b200_stream_t stream);

/* ids[b] = argmax over n of <x[b, :], weight[n, :]> with fp32 accumulation, ties to the lowest n: the LM head with a tied
 * embedding and its greedy sampling in one launch (triton_kernels/vocab_argmax.py:141-200); the logits are never written.
 * The decode GEMM above with an arg-max epilogue: x [M <= 32, K <= 1280] bf16, weight [N, K] bf16 contiguous, N a multiple
 * of 8, ids int64 [M]; workspace as for b200_argmax_rows (zero-filled once, left zero by every launch). */
int b200_lm_head_argmax(const void* x, int64_t x_stride, const void* weight, int64_t* ids, void* workspace, int32_t m,
                        int32_t n, int32_t k, int32_t overlap, b200_stream_t stream);

/* ids[r] = argmax over n of logits[r, n] (fp32 [rows, n], row stride in elements), ties to the lowest index: the arg-max
 * half of triton_kernels/vocab_argmax.py:141-200, for logits produced by a library GEMM.  ids is int64 [rows].
 * workspace: b200_argmax_rows_workspace_bytes() bytes, 8-byte aligned, zero-filled once (every launch leaves it zero);
 * rows <= 1024, n and row_stride multiples of 4, logits 16-byte aligned.  overlap: B200_OVERLAP_START only. */
int64_t b200_argmax_rows_workspace_bytes(void);
int b200_argmax_rows(const float* logits, int64_t row_stride, int64_t* ids, void* workspace, int32_t rows, int32_t n,
                     int32_t overlap, b200_stream_t stream);
int b200_add_rmsnorm(const void* x, int64_t x_stride_outer, int64_t x_stride_inner, int32_t inner_count,
                     const void* residual, int64_t residual_stride, const void* weight, void* sum_out, void* norm_out,
                     int32_t rows, int32_t dim, float eps, int32_t overlap, b200_stream_t stream);
int b200_swiglu(const void* gate_up, int64_t row_stride, void* out, int32_t rows, int32_t intermediate,
                int32_t overlap, b200_stream_t stream);
int b200_gdn_decode_prep(const void* qkv, int64_t qkv_stride, void* conv_state, const void* weight4, const void* a,
                         int64_t a_stride, const void* b, int64_t b_stride, const float* a_log, const void* dt_bias,
                         void* q_out, void* k_out, void* v_out, float* beta, float* g, int32_t batch, int32_t num_heads,
                         int32_t head_dim, b200_stream_t stream);
int b200_gdn_gated_rmsnorm(const void* x, const void* z, int64_t z_stride, const float* weight, void* out, int32_t rows,
                           int32_t num_heads, int32_t head_dim, b200_stream_t stream);


/* ------------------------------------------------------------------------------------------------------------------
 * Element-wise operators of the Gated-DeltaNet input pipeline and of the residual stream (one launch each, any number
 * of tokens).  bf16 tensors, fp32 math, one rounding where the reference rounds; channel counts are multiples of 8,
 * pointers 16-byte aligned, row strides multiples of 8 elements unless stated otherwise.
 *
 * b200_conv4_prefill: out[t,c] = silu(sum_r weight[c,r] * x[t+r-3, c]) over a packed buffer of `tokens` rows; a tap
 *   whose row lies before seq_start[t] (int32 [tokens], the first row of t's own sequence; NULL = one sequence starting
 *   at row 0) reads zero.  weight element (c, r) at weight + c*w_stride_d + r*w_stride_k.
 *   Replaces wy_lib::depthwise_causal_conv4_prefill, triton_kernels/depthwise_causal_conv4_prefill.py:108-170
 *   (kernel :18-91).
 * b200_conv4_decode: one token per sequence.  state [batch,4,channels] (contiguous, the last four conv INPUT rows) is
 *   shifted up one row, x[b] becomes row 3, out[b,c] = silu(sum_r weight4[r,c] * state[b,r,c]).
 *   Replaces wy_lib::depthwise_causal_conv4_decode, triton_kernels/depthwise_causal_conv4_decode.py:152-207
 *   (kernel :78-149).
 * b200_conv_state_from_packed_prefill: state[b,r,:] = x[cu_seqlens[b+1]-4+r, :] when that row belongs to sequence b,
 *   else zero.  Replaces wy_lib::conv_state_from_packed_prefill, triton_kernels/depthwise_causal_conv4_decode.py:332-374
 *   (kernel :254-329).
 * b200_gdn_qk_norm_gates: q_out = q * rsqrt(sum q^2 + 1e-6) * 128^-0.5 and k_out = k * rsqrt(sum k^2 + 1e-6) as
 *   contiguous bf16 [tokens,H,128]; beta = sigmoid(b) and g = -exp(a_log) * softplus(a + dt_bias) as fp32 [tokens,H].
 *   q, k [tokens,H,128] with token / head strides (multiples of 4, 8-byte aligned); a, b [tokens,H] bf16 with a token
 *   stride.  Replaces wy_lib::gdn_qk_norm_gates, triton_kernels/gdn_qk_norm_gates.py:128-200 (kernel :14-114).
 * b200_embedding_gather: out[t,:] = table[ids[t],:] (ids int32 or int64 [tokens], table [V,dim] contiguous).
 *   Replaces wy_lib::embedding_gather, triton_kernels/embedding_gather.py:62-100 (kernel :14-49).
 * b200_residual_add: out[i] = bf16(x[i] + residual[i]) over `count` contiguous elements.
 *   Replaces wy_lib::residual_add, triton_kernels/residual_add.py:23-50 (kernel :7-20).
 * b200_swiglu_pair: b200_swiglu for gate and up given as two [rows,width] matrices with their own row strides
 *   (triton_kernels/swiglu.py:75-110, kernel :17-59). */
int b200_conv4_prefill(const void* x, int64_t x_stride_t, const void* weight, int64_t w_stride_d, int64_t w_stride_k,
                       const int32_t* seq_start, void* out, int64_t out_stride_t, int32_t tokens, int32_t channels,
                       b200_stream_t stream);
int b200_conv4_decode(const void* x, int64_t x_stride_b, void* state, const void* weight4, void* out,
                      int64_t out_stride_b, int32_t batch, int32_t channels, b200_stream_t stream);
int b200_conv_state_from_packed_prefill(void* state, const void* x, int64_t x_stride_t, const int32_t* cu_seqlens,
                                        int32_t batch, int32_t channels, b200_stream_t stream);
int b200_gdn_qk_norm_gates(const void* q, int64_t q_stride_t, int64_t q_stride_h, const void* k, int64_t k_stride_t,
                           int64_t k_stride_h, const void* a, int64_t a_stride_t, const void* b, int64_t b_stride_t,
                           const float* a_log, const void* dt_bias, void* q_out, void* k_out, float* beta, float* g,
                           int32_t tokens, int32_t num_heads, int32_t head_dim, b200_stream_t stream);
int b200_embedding_gather(const void* ids, int32_t ids_are_int64, const void* table, void* out, int32_t tokens,
                          int32_t dim, b200_stream_t stream);
int b200_residual_add(const void* x, const void* residual, void* out, int64_t count, b200_stream_t stream);
int b200_swiglu_pair(const void* gate, int64_t gate_stride, const void* up, int64_t up_stride, void* out, int32_t rows,
                     int32_t width, b200_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* B200_ATTN_H_ */
