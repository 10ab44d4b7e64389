"""Opt-in subclass of the reference's `Qwen35Runner` that takes the fused entry points of this package.

With the `triton_kernels` drop-in alone the reference runner runs unchanged, operator by operator.  This subclass keeps
the runner, its caches (`engine/cache.py`), its page table (`engine/paging.py`) and its CUDA-graph decoder, and
replaces only the decode step's layer loop and the four mixer methods where one launch of this package does the work of a
chain of operators:

    decode_step        the layer loop of engine/runner.py:520-571 on the row-wise one-launch operators (residual add +
                       RMSNorm, projection with SwiGLU epilogue) with early starts between this package's kernels

    _forward           the prefill layer loop of engine/runner.py:602-666 with the residual adds inside the RMSNorms and
                       one gate/up projection (untraced calls)
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
        def decode_step(self, token_id, caches, trace=None):
            """engine/runner.py:520-571 with seven launches per layer instead of about fourteen: the residual add
            rides in the RMSNorm behind it, the SwiGLU is the epilogue of the gate/up projection, the mixers are the
            one-launch forms, and kernels of this package that follow one another start early (programmatic dependent
            launch).  Traced calls and contiguous (unpaged) caches take the reference's method."""
            paged = caches.block_table is not None and all(
                c is None or c.is_contiguous() for c in list(caches.k_caches) + list(caches.v_caches))
            if trace is not None or not paged:
                return super().decode_step(token_id, caches, trace)
            start, trigger, prefetch = ops.OVERLAP_START, ops.OVERLAP_TRIGGER, ops.OVERLAP_PREFETCH
            batch = token_id.shape[0]
            nh, nkv, d = self.w.num_attention_heads, self.w.num_key_value_heads, self.w.head_dim
            qd, kvd = nh * d, nkv * d

            def own(weight, swiglu=False):   # does this projection run on the package's weight-streaming kernel?
                n = weight.shape[0] // 2 if swiglu else weight.shape[0]
                return (weight.shape[1] <= ops.SKINNY_GEMM_PAIR_MAX_K
                        and ops.skinny_gemm_supports(batch, n, weight.shape[1], swiglu))

            def then(own_next):              # only a kernel of this package in front may be told to let its successor in
                return start | trigger if own_next else start

            def proj(x, weight, flags):
                return ops.skinny_gemm(x, weight, overlap=flags) if own(weight) else gemm_2d(x, weight)

            x = R.embedding_gather(token_id, self.w.embed_tokens)
            pending = None                   # MLP output still to be added to the residual stream
            for i, layer in enumerate(self.w.layers):
                gdn = isinstance(layer, R.GDNLayerWeights)
                proj_w = layer.in_proj_fused if gdn else layer.qkvg_fused
                out_w = layer.out_proj if gdn else layer.o_proj
                own_proj, own_out = own(proj_w), own(out_w)
                own_mlp, own_down = own(layer.mlp.gate_up, True), own(layer.mlp.down_proj)
                if pending is None:
                    h = ops.add_rmsnorm(x, layer.input_layernorm, self.eps, overlap=then(own_proj))
                else:
                    x, h = ops.add_rmsnorm(pending, layer.input_layernorm, self.eps, residual=x, overlap=then(own_proj))
                fused = proj(h, proj_w, then(True))
                if gdn:
                    mixed_in = ops.gdn_decode_fused(fused, caches.conv_states[i], layer.conv1d_decode, layer.a_log,
                                                    layer.dt_bias, layer.norm, caches.recurrent_states[i],
                                                    self.w.linear_num_heads, overlap=then(own_out) | prefetch)
                else:
                    q = fused[:, :qd].view(batch, nh, d)
                    k = fused[:, 2 * qd: 2 * qd + kvd].view(batch, nkv, d)
                    v = fused[:, 2 * qd + kvd:].view(batch, nkv, d)
                    mixed_in = ops.fused_decode_attention(q, k, v, fused[:, qd: 2 * qd], caches.k_caches[i],
                                                          caches.v_caches[i], caches.block_table, caches.pos,
                                                          self.inv_freq, self.w.rotary_dim, self._fused_ws,
                                                          overlap=then(own_out) | (prefetch if own_proj else 0),
                                                          q_norm_weight=layer.q_norm, k_norm_weight=layer.k_norm,
                                                          eps=self.eps)
                mixed = proj(mixed_in, out_w, then(True))
                x, h = ops.add_rmsnorm(mixed, layer.post_attention_layernorm, self.eps, residual=x,
                                       overlap=then(own_mlp))
                if own_mlp:
                    act = ops.skinny_gemm(h, layer.mlp.gate_up, overlap=then(own_down), swiglu=True)
                else:
                    gate_up = gemm_2d(h, layer.mlp.gate_up)
                    inter = layer.mlp.down_proj.shape[1]
                    act = R.swiglu(gate_up[:, :inter], gate_up[:, inter:])
                pending = proj(act, layer.mlp.down_proj, then(True))
            _, h = ops.add_rmsnorm(pending, self.w.norm, self.eps, residual=x, overlap=start)
            return h

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
        def _forward(self, input_ids, pos, trace, trace_layers, caches=None, seq=0, packed=None):
            """engine/runner.py:602-666 for untraced calls: the residual adds ride in the RMSNorms behind them, gate and
            up are one projection and the SwiGLU reads its two halves in place; the mixers are the runner's own methods
            (overridden below for packed batches)."""
            if trace is not None:
                return super()._forward(input_ids, pos, trace, trace_layers, caches=caches, seq=seq, packed=packed)
            x = R.embedding_gather(input_ids, self.w.embed_tokens)
            pending = None                   # MLP output still to be added to the residual stream
            for i, layer in enumerate(self.w.layers):
                tag = f"layer{i:02d}"
                if pending is None:
                    h = ops.add_rmsnorm(x, layer.input_layernorm, self.eps)
                else:
                    x, h = ops.add_rmsnorm(pending, layer.input_layernorm, self.eps, residual=x)
                if isinstance(layer, R.GDNLayerWeights):
                    if caches is None:
                        gdn_fill = None
                    elif packed is None:
                        gdn_fill = (caches.conv_states[i][seq], caches.recurrent_states[i][seq])
                    else:
                        gdn_fill = (caches.conv_states[i], caches.recurrent_states[i])
                    h = self._gdn(h, layer, None, tag, fill=gdn_fill, packed=packed)
                else:
                    h = self._attention(
                        h, layer, pos, None, tag,
                        fill=None if caches is None else (caches.k_caches[i], caches.v_caches[i]),
                        block_table=None if caches is None or not caches.paged
                        else (caches.block_table if packed is not None else caches.block_table[seq]),
                        packed=packed,
                    )
                x, h = ops.add_rmsnorm(h, layer.post_attention_layernorm, self.eps, residual=x)
                inter = layer.mlp.down_proj.shape[1]
                act = ops.swiglu_fused(gemm_2d(h, layer.mlp.gate_up), inter)
                pending = gemm_2d(act, layer.mlp.down_proj)
            _, x = ops.add_rmsnorm(pending, self.w.norm, self.eps, residual=x)
            return x

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
