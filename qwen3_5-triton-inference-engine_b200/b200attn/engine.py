"""Whole-model stepping around the CUDA operators of this package: a compact mirror of the reference runner's packed
prefill and batched decode (engine/runner.py:212-571) for the Qwen3.5-0.8B architecture - 24 layers, three
Gated-DeltaNet layers then one full-attention layer, SwiGLU MLP, tied embedding / LM head.

The attention and Gated-DeltaNet work runs on the fused operators (`fused_prefill_attention`,
`gdn_chunked_prefill_packed`, `fused_decode_attention`, `gdn_recurrent_decode`); everything else (projections, norms,
conv, gates, MLP, argmax) is the PyTorch glue of `glue.py`.  State per replica: paged KV pools and one block table
(engine/cache.py:51-217), conv and recurrent states per Gated-DeltaNet layer, a device-resident `pos`.  Decode can be
captured into one CUDA graph: every per-step quantity (token ids, positions) lives in device memory.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

from . import glue, glue_ops, ops


def _raw(op):
    """The Python body of a registered torch operator: the engine calls its own operators directly, without the
    dispatcher round trip (tens of microseconds per call) that an outside caller of `wy_lib::*` pays."""
    return getattr(op, "_init_fn", op)


_conv4_prefill = _raw(glue_ops.depthwise_causal_conv4_prefill)
_qk_norm_gates = _raw(glue_ops.gdn_qk_norm_gates)
_conv_state_pack = _raw(glue_ops.conv_state_from_packed_prefill)
_embedding_gather = _raw(glue_ops.embedding_gather)
_swiglu = _raw(glue_ops.swiglu)


@dataclass(frozen=True)
class ModelConfig:
    hidden: int = 1024
    num_layers: int = 24
    full_attention_interval: int = 4      # layers 3, 7, 11, ... are full attention
    num_q_heads: int = 8
    num_kv_heads: int = 2
    head_dim: int = 256
    rotary_dim: int = 64
    rope_theta: float = 1e7
    gdn_heads: int = 16
    gdn_dim: int = 128
    intermediate: int = 3584
    vocab: int = 248320
    eps: float = 1e-6

    def is_attention(self, layer: int) -> bool:
        return (layer + 1) % self.full_attention_interval == 0

    @property
    def gdn_width(self) -> int:
        return self.gdn_heads * self.gdn_dim


def random_weights(cfg: ModelConfig, seed: int, device, std: float = 0.02) -> dict:
    """Random-init weights of the architecture (N(0, std), bf16; A_log ~ U(0, 2.7) and the gated-norm weight in fp32,
    as engine/loader.py:82-153 types them).  Projections that share an input are stored fused, as the reference's
    decode path uses them (loader.py `_fuse_rows`)."""
    gen = torch.Generator(device=device).manual_seed(seed)

    def rnd(*shape, dtype=torch.bfloat16):
        return (torch.randn(*shape, generator=gen, device=device, dtype=torch.float32) * std).to(dtype)

    kd = cfg.gdn_width
    qd, kvd = cfg.num_q_heads * cfg.head_dim, cfg.num_kv_heads * cfg.head_dim
    layers = []
    for i in range(cfg.num_layers):
        layer = {"ln1": rnd(cfg.hidden), "ln2": rnd(cfg.hidden),
                 "gate_up": rnd(2 * cfg.intermediate, cfg.hidden), "down": rnd(cfg.hidden, cfg.intermediate)}
        if cfg.is_attention(i):
            layer.update(kind="attention", qkvg=rnd(2 * qd + 2 * kvd, cfg.hidden), q_norm=rnd(cfg.head_dim),
                         k_norm=rnd(cfg.head_dim), o_proj=rnd(cfg.hidden, qd))
        else:
            conv = rnd(3 * kd, 4)
            layer.update(kind="gdn", in_proj=rnd(4 * kd + 2 * cfg.gdn_heads, cfg.hidden), conv=conv,
                         conv4=conv.t().contiguous(),
                         a_log=torch.rand(cfg.gdn_heads, generator=gen, device=device) * 2.7,
                         dt_bias=rnd(cfg.gdn_heads), norm=1.0 + rnd(cfg.gdn_dim, dtype=torch.float32),
                         out_proj=rnd(cfg.hidden, kd))
        layers.append(layer)
    return {"embed": rnd(cfg.vocab, cfg.hidden), "norm": rnd(cfg.hidden), "layers": layers}


class Engine:
    """One replica: weights, caches and the two entry points `prefill` and `step`."""

    def __init__(self, cfg: ModelConfig, weights: dict, batch: int, max_context: int, device, page_seed: int = 0,
                 fused_glue: bool = True, on_demand_pages: bool = False, num_pages: int | None = None):
        """fused_glue: run the row-wise operators of a decode step (residual + RMSNorm, SwiGLU, conv + q/k norms +
        gates, gated RMSNorm) as this package's single-launch kernels; False keeps them as eager PyTorch (glue.py).
        on_demand_pages: KV pages come from a shared pool of `num_pages` (default: enough for every slot at
        `max_context`) as sequences grow (`serving.PageAllocator`), the `batch` sequences are independent SLOTS that
        `prefill_slots` fills one group at a time, and `set_active` masks the idle ones - what `ContinuousBatcher`
        drives.  Without it every slot owns its pages from the start, as the reference reserves them
        (engine/cache.py:154-159)."""
        self.cfg, self.w, self.batch, self.device = cfg, weights, batch, torch.device(device)
        self.fused_glue = fused_glue
        pages_per_seq = (max_context + ops.PAGE_SIZE - 1) // ops.PAGE_SIZE
        self.pages = None
        self.active = None
        if on_demand_pages:
            from .serving import PageAllocator
            num_pages = batch * pages_per_seq + 1 if num_pages is None else num_pages
            self.pages = PageAllocator(num_pages, batch, pages_per_seq, device=self.device)
            self.block_table = self.pages.block_table
            self.active = torch.ones(batch, dtype=torch.int64, device=self.device)   # 1 = the slot decodes
        else:
            num_pages = batch * pages_per_seq
            perm = torch.randperm(num_pages, generator=torch.Generator().manual_seed(page_seed))
            self.block_table = perm.view(batch, pages_per_seq).to(torch.int32).to(self.device)
        self.max_context = pages_per_seq * ops.PAGE_SIZE
        self.pos = torch.zeros(batch, dtype=torch.int64, device=self.device)
        self.kv, self.conv_state, self.rec_state = {}, {}, {}
        for i in range(cfg.num_layers):
            if cfg.is_attention(i):
                self.kv[i] = ops.allocate_paged_kv_cache(num_pages, cfg.num_kv_heads, cfg.head_dim, device=self.device)
            else:
                self.conv_state[i] = torch.zeros(batch, 4, 3 * cfg.gdn_width, dtype=torch.bfloat16, device=self.device)
                self.rec_state[i] = torch.zeros(batch, cfg.gdn_heads, cfg.gdn_dim, cfg.gdn_dim, dtype=torch.float32,
                                                device=self.device)
        self.workspace = ops.fused_decode_workspace(self.device)
        self.argmax_ws = ops.argmax_workspace(self.device)
        r = cfg.rotary_dim
        self.inv_freq = (1.0 / (cfg.rope_theta ** (torch.arange(0, r, 2, dtype=torch.float32) / r))).to(self.device)
        self.tok = torch.zeros(batch, dtype=torch.int64, device=self.device)   # input of the next step
        self.graph = None
        self._warmed = False     # an eager decode step has run (first-call set-up of the kernels is done)

    # ------------------------------------------------------------------------------------------------ shared pieces
    def _streams_weight(self, weight, swiglu: bool = False) -> bool:
        """Whether a projection of `batch` rows by this weight runs on the package's weight-streaming kernel."""
        n = weight.shape[0] // 2 if swiglu else weight.shape[0]
        # K > 4096 would take the chunked wide-K form, which is slower than cuBLAS (11.0 against 8.6 us at K = 3584
        # when forced); up to 4096 the CTA-pair form is faster (4.4 / 5.9 against 5.6 / 8.1 us at K = 2048 / 3584)
        return (self.fused_glue and weight.shape[1] <= ops.SKINNY_GEMM_PAIR_MAX_K
                and ops.skinny_gemm_supports(self.batch, n, weight.shape[1], swiglu))

    def _proj(self, x, weight, overlap: int = 0):
        """Projection of the hidden state: the weight-streaming kernel for decode-sized batches, cuBLAS otherwise."""
        if x.shape[0] == self.batch and self._streams_weight(weight):
            return ops.skinny_gemm(x, weight, overlap=overlap)
        return glue.gemm_2d(x, weight)

    def _norm(self, x, weight):
        if self.fused_glue:
            return ops.add_rmsnorm(x, weight, self.cfg.eps)
        return glue.qwen_rmsnorm(x, weight, self.cfg.eps)

    def _mlp(self, x, layer):
        cfg = self.cfg
        gate_up = glue.gemm_2d(self._norm(x, layer["ln2"]), layer["gate_up"])
        if self.fused_glue:
            h = ops.swiglu_fused(gate_up, cfg.intermediate)
        else:
            h = glue.swiglu(gate_up[:, : cfg.intermediate], gate_up[:, cfg.intermediate:])
        return glue.residual_add(glue.gemm_2d(h, layer["down"]), x)

    def _split_gdn(self, fused):
        kd, heads = self.cfg.gdn_width, self.cfg.gdn_heads
        return (fused[:, : 3 * kd], fused[:, 3 * kd: 4 * kd], fused[:, 4 * kd: 4 * kd + heads],
                fused[:, 4 * kd + heads:])

    def _split_attention(self, fused):
        cfg = self.cfg
        qd, kvd = cfg.num_q_heads * cfg.head_dim, cfg.num_kv_heads * cfg.head_dim
        n = fused.shape[0]
        q = self._norm(fused[:, :qd].view(n, cfg.num_q_heads, cfg.head_dim), self._cur["q_norm"])
        k = self._norm(fused[:, 2 * qd: 2 * qd + kvd].view(n, cfg.num_kv_heads, cfg.head_dim), self._cur["k_norm"])
        v = fused[:, 2 * qd + kvd:].view(n, cfg.num_kv_heads, cfg.head_dim)
        return q, k, v, fused[:, qd: 2 * qd]

    def _head(self, x):
        return glue.lm_head_argmax(self._norm(x, self.w["norm"]), self.w["embed"], last_only=False)

    # ------------------------------------------------------------------------------------------------------ prefill
    @torch.no_grad()
    def prefill(self, prompts: list[list[int]]) -> torch.Tensor:
        """Packed varlen prefill of `batch` prompts (engine/runner.py:212-405 with a PackedBatch); fills every cache,
        sets pos, returns the first generated token of each sequence (int64 [B]) and leaves it in `self.tok`."""
        assert len(prompts) == self.batch
        if self.pages is not None:
            for slot, prompt in enumerate(prompts):
                self.pages.release(slot)
                self.pages.ensure(slot, len(prompt) + 1)
        return self._prefill(prompts, None)

    @torch.no_grad()
    def prefill_slots(self, slots: list[int], prompts: list[list[int]]) -> torch.Tensor:
        """Packed prefill of `prompts` into the given slots only (their pages must already be there: the caller is the
        batcher, which calls `pages.ensure` first); the other slots keep their state.  Returns the first generated
        token of each prompt (int64 [len(slots)]) and leaves them in `self.tok[slots]`."""
        assert self.pages is not None, "slot-wise prefill needs on_demand_pages=True"
        assert len(slots) == len(prompts) and len(set(slots)) == len(slots)
        assert all(0 <= s < self.batch for s in slots)
        return self._prefill(prompts, torch.tensor(slots, dtype=torch.int64, device=self.device))

    def set_active(self, mask) -> None:
        """Which slots decode (host list of bools).  An idle slot still rides along in the step's launches - the batch
        dimension of a captured graph is fixed - but its position is forced back to zero after every step and its page
        table row points at the spare page, so nothing it writes is ever read."""
        assert self.active is not None and len(mask) == self.batch
        self.active.copy_(torch.tensor([1 if m else 0 for m in mask], dtype=torch.int64), non_blocking=True)

    def _prefill(self, prompts: list[list[int]], slots) -> torch.Tensor:
        cfg = self.cfg
        assert all(0 < len(p) <= self.max_context for p in prompts)
        lengths = [len(p) for p in prompts]
        table = self.block_table if slots is None else self.block_table.index_select(0, slots)

        def put(dst, src):          # write a per-sequence result into all slots, or into the chosen ones
            if slots is None:
                dst.copy_(src)
            else:
                dst.index_copy_(0, slots, src.to(dst.dtype))
        # ids, position inside the sequence and first packed row of the sequence (runner.py:136) for every token, built
        # on the host and sent as one int32 [3, T] array
        lens = np.asarray(lengths, dtype=np.int64)
        first_row = np.repeat(np.cumsum(lens) - lens, lens)
        host = np.empty((3, int(lens.sum())), dtype=np.int32)
        host[0] = np.fromiter((t for p in prompts for t in p), dtype=np.int64, count=host.shape[1])
        host[1] = np.arange(host.shape[1]) - first_row
        host[2] = first_row
        ids, pos_in_seq, seq_start = torch.from_numpy(host).to(self.device).unbind(0)
        cu, max_len = ops.build_cu_seqlens(lengths, device=self.device)
        total, heads, dim = ids.numel(), cfg.gdn_heads, cfg.gdn_dim
        if not self.fused_glue:
            assert slots is None, "slot-wise prefill runs on the single-launch operators only"
            return self._prefill_eager_glue(ids, cu, max_len, pos_in_seq, seq_start, lengths)
        # every operator between the projections is one launch of this package (cuBLAS for the prompt-sized GEMMs)
        x = _embedding_gather(ids, self.w["embed"])
        pending = None                                   # MLP output still to be added to the residual stream
        for i, layer in enumerate(self.w["layers"]):
            self._cur = layer
            if pending is None:
                h = ops.add_rmsnorm(x, layer["ln1"], cfg.eps)
            else:
                x, h = ops.add_rmsnorm(pending, layer["ln1"], cfg.eps, residual=x)
            if layer["kind"] == "gdn":
                qkv, z, a, b = self._split_gdn(glue.gemm_2d(h, layer["in_proj"]))
                conv = _conv4_prefill(qkv, layer["conv"], seq_start)
                kd = cfg.gdn_width
                q = conv[:, :kd].view(total, heads, dim)
                k = conv[:, kd: 2 * kd].view(total, heads, dim)
                v = conv[:, 2 * kd:].view(total, heads, dim)
                q_n, k_n, beta, g = _qk_norm_gates(q, k, a, b, layer["a_log"], layer["dt_bias"])
                if slots is None:                        # every slot: the kernel writes the cache's own states
                    core, _ = ops.gdn_chunked_prefill_packed(q_n, k_n, v, beta, g, cu, state_out=self.rec_state[i])
                    _conv_state_pack(self.conv_state[i], qkv, cu)
                else:
                    core, state = ops.gdn_chunked_prefill_packed(q_n, k_n, v, beta, g, cu)
                    put(self.rec_state[i], state)
                    conv_rows = torch.empty((len(prompts),) + tuple(self.conv_state[i].shape[1:]), dtype=torch.bfloat16,
                                            device=self.device)
                    _conv_state_pack(conv_rows, qkv, cu)
                    put(self.conv_state[i], conv_rows)
                normed = ops.gdn_gated_rmsnorm_fused(core, z, layer["norm"])
                mixed = glue.gemm_2d(normed, layer["out_proj"])
            else:
                q, k, v, gate = self._split_attention(glue.gemm_2d(h, layer["qkvg"]))
                k_cache, v_cache = self.kv[i]
                ctx = ops.fused_prefill_attention(q, k, v, gate, k_cache, v_cache, table, cu, pos_in_seq,
                                                  self.inv_freq, cfg.rotary_dim, max_len)
                mixed = glue.gemm_2d(ctx, layer["o_proj"])
            x, h = ops.add_rmsnorm(mixed, layer["ln2"], cfg.eps, residual=x)
            gate_up = glue.gemm_2d(h, layer["gate_up"])
            pending = glue.gemm_2d(_swiglu(gate_up[:, : cfg.intermediate], gate_up[:, cfg.intermediate:]), layer["down"])
        x = glue.residual_add(pending, x)
        last = x.index_select(0, cu[1:].long() - 1)
        first = self._head(last)
        put(self.pos, torch.tensor(lengths, dtype=torch.int64, device=self.device))
        put(self.tok, first)
        return first.clone()


    def _prefill_eager_glue(self, ids, cu, max_len, pos_in_seq, seq_start, lengths):
        """The same prefill with the operators around the path as eager PyTorch (glue.py); for comparisons."""
        cfg = self.cfg
        total, heads, dim = ids.numel(), cfg.gdn_heads, cfg.gdn_dim
        x = glue.embedding_gather(ids, self.w["embed"])
        for i, layer in enumerate(self.w["layers"]):
            self._cur = layer
            h = self._norm(x, layer["ln1"])
            if layer["kind"] == "gdn":
                qkv, z, a, b = self._split_gdn(glue.gemm_2d(h, layer["in_proj"]))
                conv = glue.depthwise_causal_conv4_prefill(qkv, layer["conv"], seq_start)
                kd = cfg.gdn_width
                q = conv[:, :kd].view(total, heads, dim)
                k = conv[:, kd: 2 * kd].view(total, heads, dim)
                v = conv[:, 2 * kd:].view(total, heads, dim)
                q_n, k_n, beta, g = glue.gdn_qk_norm_gates(q, k, a, b, layer["a_log"], layer["dt_bias"])
                core, state = ops.gdn_chunked_prefill_packed(q_n, k_n, v, beta, g, cu)
                self.rec_state[i].copy_(state)
                glue.conv_state_from_packed_prefill(self.conv_state[i], qkv, cu)
                if self.fused_glue:
                    normed = ops.gdn_gated_rmsnorm_fused(core, z, layer["norm"])
                else:
                    normed = glue.gdn_gated_rmsnorm(core, z.reshape(total, heads, dim), layer["norm"]).view(total, kd)
                mixed = glue.gemm_2d(normed, layer["out_proj"])
            else:
                q, k, v, gate = self._split_attention(glue.gemm_2d(h, layer["qkvg"]))
                k_cache, v_cache = self.kv[i]
                ctx = ops.fused_prefill_attention(q, k, v, gate, k_cache, v_cache, self.block_table, cu, pos_in_seq,
                                                  self.inv_freq, cfg.rotary_dim, max_len)
                mixed = glue.gemm_2d(ctx, layer["o_proj"])
            x = self._mlp(glue.residual_add(mixed, x), layer)
        last = x.index_select(0, cu[1:].long() - 1)
        self.pos.copy_(torch.tensor(lengths, dtype=torch.int64))
        self.tok.copy_(self._head(last))
        return self.tok.clone()

    # ------------------------------------------------------------------------------------------------------- decode
    @torch.no_grad()
    def _decode(self, tok: torch.Tensor) -> torch.Tensor:
        """One token per sequence (engine/runner.py:408-571): returns the next token ids and advances pos on the
        device.  No host value changes from step to step, so the whole call can sit in a CUDA graph."""
        if self.fused_glue:
            return self._decode_fused(tok)
        cfg = self.cfg
        batch, heads, dim, kd = self.batch, cfg.gdn_heads, cfg.gdn_dim, cfg.gdn_width
        x = glue.embedding_gather(tok, self.w["embed"])
        for i, layer in enumerate(self.w["layers"]):
            self._cur = layer
            h = glue.qwen_rmsnorm(x, layer["ln1"], cfg.eps)
            if layer["kind"] == "gdn":
                qkv, z, a, b = self._split_gdn(glue.gemm_2d(h, layer["in_proj"]))
                conv = glue.depthwise_causal_conv4_decode(qkv, self.conv_state[i], layer["conv4"])
                q = conv[:, :kd].view(batch, heads, dim)
                k = conv[:, kd: 2 * kd].view(batch, heads, dim)
                v = conv[:, 2 * kd:].view(batch, heads, dim)
                q_n, k_n, beta, g = glue.gdn_qk_norm_gates(q, k, a, b, layer["a_log"], layer["dt_bias"])
                core = ops.gdn_recurrent_decode(q_n, k_n, v, beta, g, self.rec_state[i])
                normed = glue.gdn_gated_rmsnorm(core, z.reshape(batch, heads, dim), layer["norm"])
                mixed = glue.gemm_2d(normed.view(batch, kd), layer["out_proj"])
            else:
                q, k, v, gate = self._split_attention(glue.gemm_2d(h, layer["qkvg"]))
                k_cache, v_cache = self.kv[i]
                ctx = ops.fused_decode_attention(q, k, v, gate, k_cache, v_cache, self.block_table, self.pos,
                                                 self.inv_freq, cfg.rotary_dim, self.workspace)
                mixed = glue.gemm_2d(ctx, layer["o_proj"])
            x = self._mlp(glue.residual_add(mixed, x), layer)
        nxt = self._head(x)
        self.pos.add_(1)
        if self.active is not None:
            self.pos.mul_(self.active)
        return nxt

    def _decode_fused(self, tok: torch.Tensor) -> torch.Tensor:
        """The same step with every row-wise operator as one launch: seven launches per layer (norm, projection, mixer
        with its head norms inside, output projection, norm, gate/up projection with the SwiGLU as its epilogue, down
        projection).  The residual add after a layer's MLP is fused into the next layer's input norm.  Kernels of this
        package that follow one another start early (programmatic dependent launch: weights and states stream in while
        the predecessor finishes); a kernel in front of a cuBLAS or PyTorch kernel never triggers early."""
        cfg = self.cfg
        batch, heads = self.batch, cfg.gdn_heads
        qd, kvd = cfg.num_q_heads * cfg.head_dim, cfg.num_kv_heads * cfg.head_dim
        start, trigger, prefetch = ops.OVERLAP_START, ops.OVERLAP_TRIGGER, ops.OVERLAP_PREFETCH

        def then(own_next: bool) -> int:                 # flags of a kernel whose successor is (not) one of ours
            return start | trigger if own_next else start

        x = _embedding_gather(tok, self.w["embed"])      # this package's kernel: the norm behind it may start early
        pending = None                                   # MLP output still to be added to the residual stream
        for i, layer in enumerate(self.w["layers"]):
            gdn = layer["kind"] == "gdn"
            proj_w = layer["in_proj"] if gdn else layer["qkvg"]
            out_w = layer["out_proj"] if gdn else layer["o_proj"]
            own_proj, own_out = self._streams_weight(proj_w), self._streams_weight(out_w)
            own_mlp, own_down = self._streams_weight(layer["gate_up"], swiglu=True), self._streams_weight(layer["down"])
            if pending is None:
                h = ops.add_rmsnorm(x, layer["ln1"], cfg.eps, overlap=then(own_proj))
            else:
                x, h = ops.add_rmsnorm(pending, layer["ln1"], cfg.eps, residual=x, overlap=then(own_proj))
            fused = self._proj(h, proj_w, then(True))
            if gdn:
                mixed_in = ops.gdn_decode_fused(fused, self.conv_state[i], layer["conv4"], layer["a_log"],
                                                layer["dt_bias"], layer["norm"], self.rec_state[i], heads,
                                                overlap=then(own_out) | prefetch)
            else:
                # the q / k head norms run inside the attention kernel, which starts behind the projection
                q = fused[:, :qd].view(batch, cfg.num_q_heads, cfg.head_dim)
                k = fused[:, 2 * qd: 2 * qd + kvd].view(batch, cfg.num_kv_heads, cfg.head_dim)
                v = fused[:, 2 * qd + kvd:].view(batch, cfg.num_kv_heads, cfg.head_dim)
                k_cache, v_cache = self.kv[i]
                mixed_in = ops.fused_decode_attention(q, k, v, fused[:, qd: 2 * qd], k_cache, v_cache, self.block_table,
                                                      self.pos, self.inv_freq, cfg.rotary_dim, self.workspace,
                                                      overlap=then(own_out) | (prefetch if own_proj else 0),
                                                      q_norm_weight=layer["q_norm"], k_norm_weight=layer["k_norm"],
                                                      eps=cfg.eps)
            mixed = self._proj(mixed_in, out_w, then(True))
            x, h = ops.add_rmsnorm(mixed, layer["ln2"], cfg.eps, residual=x, overlap=then(own_mlp))
            if own_mlp:
                act = ops.skinny_gemm(h, layer["gate_up"], overlap=then(own_down), swiglu=True)
            else:
                act = ops.swiglu_fused(glue.gemm_2d(h, layer["gate_up"]), cfg.intermediate, overlap=then(own_down))
            pending = self._proj(act, layer["down"], then(True))
        embed = self.w["embed"]
        own_head = (embed.shape[1] <= ops.SKINNY_GEMM_MAX_K
                    and ops.skinny_gemm_supports(batch, embed.shape[0], embed.shape[1]))
        _, h = ops.add_rmsnorm(pending, self.w["norm"], cfg.eps, residual=x, overlap=then(own_head))
        if own_head:   # tied LM head and greedy sampling in one launch; the logits are never written
            # the ids go straight into `tok` when it is the engine's own token buffer (read only by the gather at the
            # top of the step): no copy kernel behind the step
            in_place = tok.data_ptr() == self.tok.data_ptr() and tok.dtype == torch.int64 and tok.is_contiguous()
            nxt = ops.lm_head_argmax(h, embed, self.argmax_ws, out=tok if in_place else None, overlap=start)
        else:          # fp32 logits from cuBLAS, arg-max (lowest index on ties) in one launch
            nxt = glue.lm_head_argmax(h, embed, last_only=False,
                                      argmax=lambda logits: ops.argmax_rows(logits, self.argmax_ws, overlap=start))
        self.pos.add_(1)
        if self.active is not None:
            self.pos.mul_(self.active)       # idle slots stay at position 0 (and on the spare page)
        return nxt

    def capture(self) -> None:
        """Capture one decode step (read self.tok, write the next ids back into self.tok) into a CUDA graph.
        At least one eager `step()` must have run before: the first call of several kernels does per-device set-up
        (shared-memory limits, symbol addresses, workspaces) that must not happen under stream capture."""
        assert self._warmed, "run one eager step() before capture(): first calls do set-up that cannot be captured"
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                self._advance()
        torch.cuda.current_stream(self.device).wait_stream(side)
        self.graph = graph

    def step(self) -> torch.Tensor:
        """Advance every sequence by one token; returns the device tensor holding the new ids (valid until the next
        step)."""
        if self.graph is not None:
            self.graph.replay()
        else:
            self._advance()
            self._warmed = True
        return self.tok

    def _advance(self) -> None:
        nxt = self._decode(self.tok)
        if nxt.data_ptr() != self.tok.data_ptr():        # a step that did not write the ids in place
            self.tok.copy_(nxt)
