"""Opt-in subclass of the reference's `Qwen35Runner` that takes the fused entry points of this package.

With the `triton_kernels` drop-in alone the reference runner runs unchanged, operator by operator.  This subclass keeps
the runner, its caches (`engine/cache.py`), its page table (`engine/paging.py`) and its CUDA-graph decoder, and
replaces only the four mixer methods where one launch of this package does the work of a chain of operators:

    _attention_decode  fused_decode_attention: q/k head norms + partial RoPE + KV append + paged attention + gate
                       (engine/runner.py:444-518 is eleven operator calls)
    _gdn_decode        gdn_decode_fused: conv step + q/k norms + gates + delta-rule step + gated norm
                       (engine/runner.py:408-442)
    _attention         packed prefill: fused_prefill_attention (RoPE + attention + gate + paged scatter,
                       engine/runner.py:339-384); other calls fall through to the reference's method
    _gdn               packed prefill: the chunk-64 tensor-core kernel with cu_seqlens instead of the token-serial
                       recurrence the reference must use for packed batches (engine/runner.py:263-271)

The reference engine is imported, not copied: put the reference checkout (or baseline/_ref) on `sys.path` AFTER
importing this package's `triton_kernels`, then call `fast_runner_class()`.
"""
from __future__ import annotations

import torch

from . import glue_ops, ops


def fast_runner_class():
    """Build the subclass against whatever `engine.runner` is importable (the reference's, unmodified)."""
    import engine.runner as R

    gemm_2d = R.gemm_2d   # the drop-in operator the reference module already imported

    class FastRunner(R.Qwen35Runner):
        """`Qwen35Runner` with the fused decode / packed-prefill mixers of libb200attn.so."""

        def __init__(self, weights, compile: bool = False):
            super().__init__(weights, compile=compile)
            self._fused_ws = ops.fused_decode_workspace(self.device)

        # ------------------------------------------------------------------------------------------- decode
        def _attention_decode(self, h, w, k_cache, v_cache, pos, scratch, block_table=None):
            if block_table is None or not (k_cache.is_contiguous() and v_cache.is_contiguous()):
                return super()._attention_decode(h, w, k_cache, v_cache, pos, scratch, block_table)
            nh, nkv, d = self.w.num_attention_heads, self.w.num_key_value_heads, self.w.head_dim
            batch = h.shape[0]
            fused = gemm_2d(h, w.qkvg_fused)                                   # [B, 2*nh*d + 2*nkv*d]
            qd, kd = nh * d, nkv * d
            q = fused[:, :qd].view(batch, nh, d)
            gate = fused[:, qd: 2 * qd]
            k = fused[:, 2 * qd: 2 * qd + kd].view(batch, nkv, d)
            v = fused[:, 2 * qd + kd:].view(batch, nkv, d)
            ctx = ops.fused_decode_attention(q, k, v, gate, k_cache, v_cache, block_table, pos, self.inv_freq,
                                             self.w.rotary_dim, self._fused_ws, q_norm_weight=w.q_norm,
                                             k_norm_weight=w.k_norm, eps=self.eps)
            return gemm_2d(ctx, w.o_proj)

        def _gdn_decode(self, h, w, conv_state, recurrent_state):
            heads = self.w.linear_num_heads
            fused = gemm_2d(h, w.in_proj_fused)                                # [B, q|k|v|z|a|b]
            mixed = ops.gdn_decode_fused(fused, conv_state, w.conv1d_decode, w.a_log, w.dt_bias, w.norm, recurrent_state,
                                         heads)
            return gemm_2d(mixed, w.out_proj)

        # ------------------------------------------------------------------------------------------ prefill
        def _attention(self, h, w, pos, trace, tag, fill=None, block_table=None, packed=None):
            if packed is None or fill is None or block_table is None or trace is not None:
                return super()._attention(h, w, pos, trace, tag, fill=fill, block_table=block_table, packed=packed)
            token_num = h.shape[0]
            nh, nkv, d = self.w.num_attention_heads, self.w.num_key_value_heads, self.w.head_dim
            q = R.qwen_rmsnorm(gemm_2d(h, w.q_proj_q).view(token_num, nh, d), w.q_norm, self.eps)
            gate = gemm_2d(h, w.q_proj_gate)
            k = R.qwen_rmsnorm(gemm_2d(h, w.k_proj).view(token_num, nkv, d), w.k_norm, self.eps)
            v = gemm_2d(h, w.v_proj).view(token_num, nkv, d)
            k_cache, v_cache = fill
            ctx = ops.fused_prefill_attention(q, k, v, gate, k_cache, v_cache, block_table, packed.cu_seqlens,
                                              packed.position_ids, self.inv_freq, self.w.rotary_dim, packed.max_seqlen)
            return gemm_2d(ctx, w.o_proj)

        def _gdn(self, h, w, trace, tag, fill=None, packed=None):
            if packed is None:
                return super()._gdn(h, w, trace, tag, fill=fill, packed=packed)
            # The reference's method, unchanged, with ONE operator swapped for the duration of the call: its packed
            # branch calls the token-serial recurrence because its chunk-64 path cannot take cu_seqlens; this
            # package's chunk-64 kernel can.
            serial = R.gdn_recurrent_prefill_sequential

            def chunked(q, k, v, beta, g, cu_seqlens=None):
                if cu_seqlens is None:
                    return serial(q, k, v, beta, g)
                return ops.gdn_chunked_prefill_packed(q, k, v, beta, g, cu_seqlens)

            R.gdn_recurrent_prefill_sequential = chunked
            try:
                return super()._gdn(h, w, trace, tag, fill=fill, packed=packed)
            finally:
                R.gdn_recurrent_prefill_sequential = serial

    return FastRunner


__all__ = ["fast_runner_class"]
_ = (glue_ops, torch)   # the drop-in operators must be registered before the reference engine is imported
