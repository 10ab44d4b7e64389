"""torch.library operators `wy_lib::*` backed by libb200attn.so.

Same operator names, schemas, argument meaning and assert-before-launch behaviour as the reference's
`triton_kernels/*.py` wrappers (each function cites the one it replaces), so `engine/runner.py`, `cache.py` and
`paging.py` of the reference can import them unchanged through the `triton_kernels` shim package next to this one.
Outputs are allocated with torch on the inputs' device; caches, state and scratch are caller-owned and
mutated in place.  Everything launches on `torch.cuda.current_stream()`; nothing synchronises.
"""
from __future__ import annotations

import math

import torch

from . import _lib

PAGE_SIZE = 16     # triton_kernels/gqa_attention_decode_paged.py:91
MAX_SPLITS = 128   # triton_kernels/gqa_attention_decode_paged.py:95
GDN_CHUNK = 64
GDN_DIM = 128      # key and value dim the Gated-DeltaNet kernels are specialised for


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)   # the handle without building a Stream object


def _stream():
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: torch.Tensor | None):
    return None if t is None else t.data_ptr()


def _inner_contiguous(t: torch.Tensor) -> torch.Tensor:
    """The C ABI wants unit stride on the last dim; anything else is materialised (never the case in the engine)."""
    return t if t.stride(-1) == 1 else t.contiguous()


def _require_cuda(*tensors):
    for t in tensors:
        if t is not None:
            assert t.is_cuda, "b200attn operators run on CUDA tensors only (there is no CPU fallback)"


# =========================================================================== paged KV cache
@torch.library.custom_op("wy_lib::paged_kv_append", mutates_args=("k_cache", "v_cache"), device_types="cuda")
def paged_kv_append(k_cache: torch.Tensor, v_cache: torch.Tensor, k_new: torch.Tensor, v_new: torch.Tensor,
                    block_table: torch.Tensor, pos: torch.Tensor) -> None:
    """Replaces triton_kernels/gqa_attention_decode_paged.py:254-305."""
    batch, num_kv_heads, head_dim = k_new.shape
    assert k_cache.shape[1] == num_kv_heads and k_cache.shape[3] == head_dim
    assert k_cache.shape[2] == PAGE_SIZE
    assert v_cache.shape == k_cache.shape
    assert k_new.shape == v_new.shape
    assert k_cache.dtype == v_cache.dtype == torch.bfloat16
    assert k_new.dtype == v_new.dtype == torch.bfloat16
    assert block_table.dtype == torch.int32 and block_table.shape[0] == batch
    assert pos.dtype == torch.int64 and pos.shape == (batch,)
    assert k_cache.stride(3) == 1 and v_cache.stride(3) == 1 and block_table.stride(1) == 1
    _require_cuda(k_cache, v_cache, k_new, v_new, block_table, pos)
    k_new, v_new, pos = _inner_contiguous(k_new), _inner_contiguous(v_new), pos.contiguous()
    _lib.call("b200_paged_kv_append", _ptr(k_cache), _ptr(v_cache), k_cache.stride(0), k_cache.stride(1),
              k_cache.stride(2), v_cache.stride(0), v_cache.stride(1), v_cache.stride(2), _ptr(k_new), k_new.stride(0),
              k_new.stride(1), _ptr(v_new), v_new.stride(0), v_new.stride(1), _ptr(block_table), block_table.stride(0),
              _ptr(pos), batch, num_kv_heads, head_dim, _stream())


@paged_kv_append.register_fake
def _(k_cache, v_cache, k_new, v_new, block_table, pos) -> None:
    return None


@torch.library.custom_op("wy_lib::paged_kv_fill_varlen", mutates_args=("k_cache", "v_cache"), device_types="cuda")
def paged_kv_fill_varlen(k_cache: torch.Tensor, v_cache: torch.Tensor, k_packed: torch.Tensor, v_packed: torch.Tensor,
                         block_table: torch.Tensor, cu_seqlens: torch.Tensor, max_seqlen: int) -> None:
    """Replaces triton_kernels/gqa_attention_decode_paged.py:492-561.  k_packed/v_packed are [H_kv, T, D] views."""
    num_kv_heads, total_tokens, head_dim = k_packed.shape
    assert v_packed.shape == k_packed.shape
    assert k_cache.shape[1] == num_kv_heads and k_cache.shape[3] == head_dim
    assert k_cache.shape[2] == PAGE_SIZE
    assert v_cache.shape == k_cache.shape
    assert k_cache.dtype == v_cache.dtype == torch.bfloat16
    assert k_packed.dtype == v_packed.dtype == torch.bfloat16
    assert block_table.dtype == torch.int32 and block_table.ndim == 2
    assert cu_seqlens.dtype == torch.int32 and cu_seqlens.ndim == 1
    batch = cu_seqlens.shape[0] - 1
    assert block_table.shape[0] == batch, (
        f"block_table has {block_table.shape[0]} rows but cu_seqlens describes {batch} sequences")
    assert block_table.shape[1] >= (max_seqlen + PAGE_SIZE - 1) // PAGE_SIZE, (
        f"page table rows hold {block_table.shape[1]} pages, too few for {max_seqlen} tokens")
    assert k_cache.stride(3) == 1 and v_cache.stride(3) == 1 and block_table.stride(1) == 1
    _require_cuda(k_cache, v_cache, k_packed, v_packed, block_table, cu_seqlens)
    k_packed, v_packed = _inner_contiguous(k_packed), _inner_contiguous(v_packed)
    cu_seqlens = cu_seqlens.contiguous()
    _lib.call("b200_paged_kv_fill_varlen", _ptr(k_cache), _ptr(v_cache), k_cache.stride(0), k_cache.stride(1),
              k_cache.stride(2), v_cache.stride(0), v_cache.stride(1), v_cache.stride(2), _ptr(k_packed),
              k_packed.stride(0), k_packed.stride(1), _ptr(v_packed), v_packed.stride(0), v_packed.stride(1),
              _ptr(block_table), block_table.stride(0), _ptr(cu_seqlens), batch, num_kv_heads, head_dim,
              int(max_seqlen), _stream())


@paged_kv_fill_varlen.register_fake
def _(k_cache, v_cache, k_packed, v_packed, block_table, cu_seqlens, max_seqlen) -> None:
    return None


# =========================================================================== paged decode attention
@torch.library.custom_op("wy_lib::paged_gqa_attention_decode_split",
                         mutates_args=("m_partial", "l_partial", "acc_partial"), device_types="cuda")
def paged_gqa_attention_decode_split(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                                     block_table: torch.Tensor, m_partial: torch.Tensor, l_partial: torch.Tensor,
                                     acc_partial: torch.Tensor, pos: torch.Tensor, seq_bucket: int) -> None:
    """Replaces triton_kernels/gqa_attention_decode_paged.py:822-891.  `seq_bucket` only keyed the reference's
    autotuner and is ignored."""
    batch, num_q_heads, head_dim = q.shape
    num_pages, num_kv_heads, page, cache_dim = k_cache.shape
    assert page == PAGE_SIZE and cache_dim == head_dim
    assert v_cache.shape == k_cache.shape
    assert q.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16
    assert block_table.dtype == torch.int32 and block_table.shape[0] == batch
    assert m_partial.shape == (batch, num_q_heads, MAX_SPLITS)
    assert l_partial.shape == (batch, num_q_heads, MAX_SPLITS)
    assert acc_partial.shape == (batch, num_q_heads, MAX_SPLITS, head_dim)
    assert m_partial.dtype == l_partial.dtype == acc_partial.dtype == torch.float32
    assert m_partial.is_contiguous() and l_partial.is_contiguous() and acc_partial.is_contiguous()
    assert pos.dtype == torch.int64 and pos.shape == (batch,)
    assert num_q_heads % num_kv_heads == 0
    assert k_cache.stride(3) == 1 and v_cache.stride(3) == 1 and block_table.stride(1) == 1
    _require_cuda(q, k_cache, v_cache, block_table, m_partial, l_partial, acc_partial, pos)
    q, pos = _inner_contiguous(q), pos.contiguous()
    _lib.call("b200_paged_decode_split", _ptr(q), q.stride(0), q.stride(1), _ptr(k_cache), _ptr(v_cache),
              k_cache.stride(0), k_cache.stride(1), k_cache.stride(2), v_cache.stride(0), v_cache.stride(1),
              v_cache.stride(2), _ptr(block_table), block_table.stride(0), _ptr(m_partial), _ptr(l_partial),
              _ptr(acc_partial), _ptr(pos), batch, num_q_heads, num_kv_heads, head_dim, _stream())


@paged_gqa_attention_decode_split.register_fake
def _(q, k_cache, v_cache, block_table, m_partial, l_partial, acc_partial, pos, seq_bucket) -> None:
    return None


@torch.library.custom_op("wy_lib::paged_gqa_attention_decode_combine", mutates_args=(), device_types="cuda")
def paged_gqa_attention_decode_combine(m_partial: torch.Tensor, l_partial: torch.Tensor, acc_partial: torch.Tensor,
                                       pos: torch.Tensor) -> torch.Tensor:
    """Replaces triton_kernels/gqa_attention_decode_paged.py:901-939."""
    batch, num_q_heads, _, head_dim = acc_partial.shape
    assert m_partial.is_contiguous() and l_partial.is_contiguous() and acc_partial.is_contiguous()
    assert pos.dtype == torch.int64 and pos.shape == (batch,)
    _require_cuda(m_partial, l_partial, acc_partial, pos)
    out = torch.empty((batch, num_q_heads, head_dim), dtype=torch.bfloat16, device=acc_partial.device)
    pos = pos.contiguous()  # kept alive until the launch is enqueued
    _lib.call("b200_paged_decode_combine", _ptr(m_partial), _ptr(l_partial), _ptr(acc_partial), _ptr(pos),
              _ptr(out), batch, num_q_heads, head_dim, _stream())
    return out


@paged_gqa_attention_decode_combine.register_fake
def _(m_partial, l_partial, acc_partial, pos) -> torch.Tensor:
    batch, num_q_heads, _, head_dim = acc_partial.shape
    return torch.empty((batch, num_q_heads, head_dim), dtype=torch.bfloat16, device=acc_partial.device)


def allocate_paged_kv_cache(num_pages: int, num_kv_heads: int, head_dim: int, *, device="cuda"):
    """`[num_pages, H_kv, PAGE, D]` bf16 K and V pools.  triton_kernels/gqa_attention_decode_paged.py:100-111."""
    shape = (num_pages, num_kv_heads, PAGE_SIZE, head_dim)
    return (torch.zeros(shape, dtype=torch.bfloat16, device=device),
            torch.zeros(shape, dtype=torch.bfloat16, device=device))


def allocate_split_scratch(num_q_heads: int, head_dim: int, *, batch: int = 1, device="cuda"):
    """(m, l, acc) split-K scratch shared by all layers.  triton_kernels/gqa_attention_decode_paged.py:591-609."""
    m = torch.zeros((batch, num_q_heads, MAX_SPLITS), dtype=torch.float32, device=device)
    l = torch.zeros((batch, num_q_heads, MAX_SPLITS), dtype=torch.float32, device=device)
    acc = torch.zeros((batch, num_q_heads, MAX_SPLITS, head_dim), dtype=torch.float32, device=device)
    return m, l, acc


def physical_rows(block_table: torch.Tensor, token_index: torch.Tensor, num_kv_heads: int) -> torch.Tensor:
    """row(t,h) = (block_table[t // PAGE] * H + h) * PAGE + t % PAGE, [T, H], all on the device.
    triton_kernels/gqa_attention_decode_paged.py:127-144."""
    logical_page = token_index // PAGE_SIZE
    slot = token_index % PAGE_SIZE
    phys = block_table.index_select(0, logical_page.to(torch.int32)).to(torch.int64)
    heads = torch.arange(num_kv_heads, device=block_table.device, dtype=torch.int64)
    return (phys[:, None] * num_kv_heads + heads[None, :]) * PAGE_SIZE + slot[:, None]


def paged_kv_fill(k_cache, v_cache, k_prefill, v_prefill, block_table) -> None:
    """Single-sequence scatter of `[H, T, D]` K/V (block_table is that sequence's row).
    triton_kernels/gqa_attention_decode_paged.py:355-375; served by the varlen kernel with cu_seqlens=[0, T]."""
    num_kv_heads, token_num, head_dim = k_prefill.shape
    assert v_prefill.shape == k_prefill.shape
    cu = torch.tensor([0, token_num], dtype=torch.int32, device=k_cache.device)
    paged_kv_fill_varlen(k_cache, v_cache, k_prefill, v_prefill, block_table.reshape(1, -1), cu, token_num)


# How `call_paged_gqa_attention_decode_triton` runs: True = for four sequences or more, one launch of the fused decode
# kernel without RoPE and gate (append + attention; `scratch` stays untouched); False = always the reference's three
# launches append -> split -> combine through `scratch` (which one or two sequences always take: three chained 2-5 us
# launches are quicker there than the fused kernel's cluster launch).
DECODE_CALL_ONE_LAUNCH = True
_decode_call_ws: dict = {}   # device index -> workspace of the one-launch form (zero-filled once, left zero by every call)


def _one_launch_decode_ok(q, k_new, v_new, k_cache, v_cache, block_table, pos) -> bool:
    """The shape and layout rules of b200_fused_decode_attention_static."""
    batch, hq, d = q.shape
    hkv = k_new.shape[1]
    return (d == 256 and hq == 4 * hkv and 8 <= batch * hkv <= 2048 and batch <= 512 and k_cache.is_contiguous()
            and v_cache.is_contiguous() and k_cache.shape[1:] == (hkv, PAGE_SIZE, d) and v_cache.shape == k_cache.shape
            and q.stride(2) == 1 and k_new.stride(2) == 1 and v_new.stride(2) == 1
            and all(t.data_ptr() % 16 == 0 for t in (q, k_new, v_new))
            and all(st % 8 == 0 for t in (q, k_new, v_new) for st in t.stride()[:2])
            and block_table.stride(1) == 1 and pos.is_contiguous())


def call_paged_gqa_attention_decode_triton(q, k_new, v_new, k_cache, v_cache, block_table, pos, scratch=None):
    """append -> attention over the pos[b]+1 cached tokens, the symbol engine/runner.py:508-510 calls
    (triton_kernels/gqa_attention_decode_paged.py:963-994; the name is kept for drop-in use, no Triton is involved).
    q and k_new arrive rotated; returns [B, H_q, D] bf16.  By default this is ONE launch of the fused decode kernel (no
    RoPE, no gate): the reference's split-K partials (4 KiB written and read per split, a third of the KV bytes at
    B = 256) never exist.  With DECODE_CALL_ONE_LAUNCH off, or for layouts the fused kernel does not take, it is the
    reference's three launches append -> split -> combine through `scratch`.  The one-launch form keeps one workspace
    per device: like the reference's runner, call it from one stream at a time."""
    if DECODE_CALL_ONE_LAUNCH and _one_launch_decode_ok(q, k_new, v_new, k_cache, v_cache, block_table, pos):
        batch, hq, d = q.shape
        hkv = k_new.shape[1]
        _require_cuda(q, k_new, v_new, k_cache, v_cache, block_table, pos)
        assert q.dtype == k_new.dtype == v_new.dtype == k_cache.dtype == v_cache.dtype == torch.bfloat16
        assert block_table.dtype == torch.int32 and pos.dtype == torch.int64 and pos.shape == (batch,)
        out = torch.empty((batch, hq, d), dtype=torch.bfloat16, device=q.device)
        ws = _decode_call_ws.get(q.device.index)
        if ws is None and not torch.cuda.is_current_stream_capturing():
            ws = _decode_call_ws[q.device.index] = fused_decode_workspace(q.device)
        if ws is None:
            # first call on this device inside a stream capture: nothing may be allocated, the library's static workspace
            # (cleared on the stream before the launch) serves instead
            _lib.call("b200_fused_decode_attention_static", _ptr(q), q.stride(0), q.stride(1), _ptr(k_new),
                      k_new.stride(0), k_new.stride(1), _ptr(v_new), v_new.stride(0), v_new.stride(1), None, 0,
                      _ptr(k_cache), _ptr(v_cache), k_cache.stride(0), k_cache.stride(1), k_cache.stride(2),
                      v_cache.stride(0), v_cache.stride(1), v_cache.stride(2), k_cache.shape[0], _ptr(block_table),
                      block_table.stride(0), _ptr(pos), None, 0, _ptr(out), batch, hq, hkv, d, _stream())
            return out
        _lib.call("b200_fused_decode_attention_ex", _ptr(q), q.stride(0), q.stride(1), _ptr(k_new), k_new.stride(0),
                  k_new.stride(1), _ptr(v_new), v_new.stride(0), v_new.stride(1), None, 0, _ptr(k_cache), _ptr(v_cache),
                  k_cache.stride(0), k_cache.stride(1), k_cache.stride(2), v_cache.stride(0), v_cache.stride(1),
                  v_cache.stride(2), k_cache.shape[0], _ptr(block_table), block_table.stride(0), _ptr(pos), None, 0,
                  _ptr(out), _ptr(ws), batch, hq, hkv, d, None, None, 1e-6, chain_flags(), 0, _stream())
        return out
    if scratch is None:
        scratch = allocate_split_scratch(q.shape[1], q.shape[2], batch=q.shape[0], device=q.device)
    m_partial, l_partial, acc_partial = scratch
    paged_kv_append(k_cache, v_cache, k_new, v_new, block_table, pos)
    hint = k_cache.shape[0] * PAGE_SIZE
    paged_gqa_attention_decode_split(q, k_cache, v_cache, block_table, m_partial, l_partial, acc_partial, pos, hint)
    return paged_gqa_attention_decode_combine(m_partial, l_partial, acc_partial, pos)


# --------------------------------------------------------------------------- fused decode (new entry point)
def fused_decode_workspace(device="cuda") -> torch.Tensor:
    """Zero-filled workspace for `fused_decode_attention` (one per stream of calls; shared by all layers)."""
    nbytes = _lib.load().b200_fused_decode_workspace_bytes()
    return torch.zeros(nbytes, dtype=torch.uint8, device=device)


def fused_decode_attention(q, k_new, v_new, gate, k_cache, v_cache, block_table, pos, inv_freq, rotary_dim,
                           workspace, out=None, overlap: int = 0, q_norm_weight=None, k_norm_weight=None,
                           eps: float = 1e-6, partition: int = 0) -> torch.Tensor:
    """RoPE(q, k_new) + append + paged attention + sigmoid gate in one launch -> [B, H_q*D] bf16.
    q [B,H_q,D], k_new/v_new [B,H_kv,D] are the post-norm, PRE-RoPE projections; gate [B, H_q*D].
    q_norm_weight / k_norm_weight (bf16 [D]): q and k_new are the RAW projections and the per-head Qwen RMSNorm
    (engine/runner.py:476-489) is applied inside the kernel - the same bytes as add_rmsnorm in front of the call.
    overlap: OVERLAP_START lets the kernel begin while its predecessor in the stream runs; OVERLAP_PREFETCH also lets it
    read pos / block_table / cache pages before that predecessor has finished (valid when it writes none of them).
    partition: 0 = the kernel picks how the KV pages are cut over the CTAs; 1 = equal page ranges per CTA (segments cut at
    a range boundary are merged through the workspace); 2 = one whole (sequence, kv head) segment per CTA (needs
    batch * H_kv <= the number of SMs); 3 = one segment per thread-block cluster, merged through distributed shared
    memory (needs batch * H_kv <= 64).  Same result up to fp32 summation order."""
    batch, num_q_heads, head_dim = q.shape
    num_kv_heads = k_new.shape[1]
    assert k_new.shape == v_new.shape == (batch, num_kv_heads, head_dim)
    assert gate.shape == (batch, num_q_heads * head_dim)
    assert q.dtype == k_new.dtype == v_new.dtype == gate.dtype == k_cache.dtype == v_cache.dtype == torch.bfloat16
    assert k_cache.shape[1:] == (num_kv_heads, PAGE_SIZE, head_dim) and v_cache.shape == k_cache.shape
    assert block_table.dtype == torch.int32 and block_table.shape[0] == batch and block_table.stride(1) == 1
    assert pos.dtype == torch.int64 and pos.shape == (batch,) and pos.is_contiguous()
    assert inv_freq.dtype == torch.float32 and inv_freq.shape == (rotary_dim // 2,) and inv_freq.is_contiguous()
    assert k_cache.is_contiguous() and v_cache.is_contiguous(), "the fused kernel reads pages by TMA: dense pools only"
    _require_cuda(q, k_new, v_new, gate, k_cache, v_cache, block_table, pos, inv_freq, workspace)
    q, k_new, v_new, gate = map(_inner_contiguous, (q, k_new, v_new, gate))
    if out is None:
        out = torch.empty((batch, num_q_heads * head_dim), dtype=torch.bfloat16, device=q.device)
    assert out.is_contiguous() and out.shape == (batch, num_q_heads * head_dim)
    for w in (q_norm_weight, k_norm_weight):
        assert w is None or (w.dtype == torch.bfloat16 and w.is_contiguous() and w.numel() == head_dim and w.device == q.device)
    _lib.call("b200_fused_decode_attention_ex", _ptr(q), q.stride(0), q.stride(1), _ptr(k_new), k_new.stride(0),
              k_new.stride(1), _ptr(v_new), v_new.stride(0), v_new.stride(1), _ptr(gate), gate.stride(0),
              _ptr(k_cache), _ptr(v_cache), k_cache.stride(0), k_cache.stride(1), k_cache.stride(2), v_cache.stride(0),
              v_cache.stride(1), v_cache.stride(2), k_cache.shape[0], _ptr(block_table), block_table.stride(0), _ptr(pos),
              _ptr(inv_freq), int(rotary_dim), _ptr(out), _ptr(workspace), batch, num_q_heads, num_kv_heads, head_dim,
              _ptr(q_norm_weight) if q_norm_weight is not None else None,
              _ptr(k_norm_weight) if k_norm_weight is not None else None, float(eps), int(overlap), int(partition),
              _stream())
    return out


# =========================================================================== rope / gate
@torch.library.custom_op("wy_lib::partial_rope", mutates_args=(), device_types="cuda")
def partial_rope(x: torch.Tensor, position_ids: torch.Tensor, inv_freq: torch.Tensor, rotary_dim: int) -> torch.Tensor:
    """Replaces triton_kernels/partial_rope.py:145-198."""
    assert x.ndim == 4
    assert x.dtype == torch.bfloat16
    assert position_ids.ndim == 2
    assert position_ids.dtype in (torch.int32, torch.int64)
    assert inv_freq.ndim == 1 and inv_freq.dtype == torch.float32
    assert x.device == position_ids.device == inv_freq.device
    batch_size, num_heads, token_num, head_dim = x.shape
    assert position_ids.shape == (batch_size, token_num)
    assert rotary_dim > 0 and rotary_dim <= head_dim and rotary_dim % 2 == 0
    assert inv_freq.shape == (rotary_dim // 2,)
    _require_cuda(x)
    x = _inner_contiguous(x)
    out = torch.empty_like(x)
    assert out.stride(3) == 1
    inv_freq = inv_freq.contiguous()  # kept alive until the launch is enqueued
    _lib.call("b200_partial_rope", _ptr(x), x.stride(0), x.stride(1), x.stride(2), _ptr(out), out.stride(0),
              out.stride(1), out.stride(2), _ptr(position_ids), int(position_ids.dtype == torch.int64),
              position_ids.stride(0), position_ids.stride(1), _ptr(inv_freq), batch_size, num_heads,
              token_num, head_dim, int(rotary_dim), _stream())
    return out


@partial_rope.register_fake
def _(x, position_ids, inv_freq, rotary_dim) -> torch.Tensor:
    return torch.empty_like(x)


@torch.library.custom_op("wy_lib::attention_gate_pack", mutates_args=(), device_types="cuda")
def attention_gate_pack(x: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
    """Replaces triton_kernels/attention_gate_pack.py:77-126."""
    assert x.ndim == 4 and gate.ndim == 4
    assert x.shape == gate.shape
    assert x.dtype == torch.bfloat16 and gate.dtype == torch.bfloat16
    assert x.device == gate.device
    batch_size, num_heads, token_num, head_dim = x.shape
    assert batch_size == 1
    assert token_num > 0
    assert head_dim > 0
    _require_cuda(x, gate)
    x, gate = _inner_contiguous(x), _inner_contiguous(gate)
    out = torch.empty((token_num, num_heads * head_dim), dtype=x.dtype, device=x.device)
    _lib.call("b200_attention_gate_pack", _ptr(x), x.stride(1), x.stride(2), _ptr(gate), gate.stride(1), gate.stride(2),
              _ptr(out), num_heads, token_num, head_dim, _stream())
    return out


@attention_gate_pack.register_fake
def _(x, gate) -> torch.Tensor:
    return torch.empty((x.shape[2], x.shape[1] * x.shape[3]), dtype=x.dtype, device=x.device)


# =========================================================================== Gated DeltaNet
def _check_gdn(q, k, v, beta, g):
    assert q.ndim == 3 and k.ndim == 3 and v.ndim == 3
    assert q.shape == k.shape
    assert q.shape[:2] == v.shape[:2]
    assert beta.ndim == 2 and g.ndim == 2
    assert beta.shape == g.shape == q.shape[:2]
    assert q.dtype == torch.bfloat16
    assert k.dtype == torch.bfloat16
    assert v.dtype == torch.bfloat16
    assert beta.dtype == torch.float32 and g.dtype == torch.float32
    assert q.device == k.device == v.device == beta.device == g.device
    _require_cuda(q)


@torch.library.custom_op("wy_lib::gdn_recurrent_decode", mutates_args=("state",), device_types="cuda")
def gdn_recurrent_decode(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, beta: torch.Tensor, g: torch.Tensor,
                         state: torch.Tensor) -> torch.Tensor:
    """Replaces triton_kernels/gdn_recurrent_prefill.py:1185-1259.  `state` [B,H,DK,DV] fp32 is updated in place."""
    _check_gdn(q, k, v, beta, g)
    assert state.dtype == torch.float32 and state.device == q.device
    batch, num_heads, key_dim = q.shape
    value_dim = v.shape[-1]
    assert state.shape == (batch, num_heads, key_dim, value_dim), (
        f"state must be [B,H,DK,DV]={(batch, num_heads, key_dim, value_dim)}, got {tuple(state.shape)}")
    assert state.stride(3) == 1 and state.stride(2) == value_dim
    q, k, v = map(_inner_contiguous, (q, k, v))
    out = torch.empty_like(v)
    assert out.stride(2) == 1
    _lib.call("b200_gdn_recurrent_decode", _ptr(q), q.stride(0), q.stride(1), _ptr(k), k.stride(0), k.stride(1),
              _ptr(v), v.stride(0), v.stride(1), _ptr(beta), beta.stride(0), beta.stride(1), _ptr(g), g.stride(0),
              g.stride(1), _ptr(state), state.stride(0), state.stride(1), _ptr(out), out.stride(0), out.stride(1),
              batch, num_heads, key_dim, value_dim, _stream())
    return out


@gdn_recurrent_decode.register_fake
def _(q, k, v, beta, g, state) -> torch.Tensor:
    return torch.empty_like(v)


@torch.library.custom_op("wy_lib::gdn_recurrent_prefill_sequential", mutates_args=(), device_types="cuda")
def gdn_recurrent_prefill_sequential(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, beta: torch.Tensor,
                                     g: torch.Tensor,
                                     cu_seqlens: torch.Tensor | None = None) -> tuple[torch.Tensor, torch.Tensor]:
    """Replaces triton_kernels/gdn_recurrent_prefill.py:1050-1145.  Returns (out [T,H,DV] bf16, state); state is
    [B,H,DK,DV] with cu_seqlens, [H,DK,DV] without."""
    _check_gdn(q, k, v, beta, g)
    token_num, num_heads, key_dim = q.shape
    value_dim = v.shape[-1]
    assert token_num > 0 and num_heads > 0
    if cu_seqlens is None:
        squeeze_state, batch = True, 1
    else:
        assert cu_seqlens.dtype == torch.int32 and cu_seqlens.ndim == 1
        assert int(cu_seqlens[-1]) == token_num, (
            f"cu_seqlens[-1]={int(cu_seqlens[-1])} does not match the {token_num} packed tokens")
        squeeze_state, batch = False, cu_seqlens.numel() - 1
        cu_seqlens = cu_seqlens.contiguous()
    q, k, v = map(_inner_contiguous, (q, k, v))
    out = torch.empty_like(v)
    assert out.stride(2) == 1
    state = torch.empty((batch, num_heads, key_dim, value_dim), dtype=torch.float32, device=q.device)
    _lib.call("b200_gdn_recurrent_prefill_sequential", _ptr(q), q.stride(0), q.stride(1), _ptr(k), k.stride(0),
              k.stride(1), _ptr(v), v.stride(0), v.stride(1), _ptr(beta), beta.stride(0), beta.stride(1), _ptr(g),
              g.stride(0), g.stride(1), _ptr(cu_seqlens), batch, token_num, _ptr(state), _ptr(out), out.stride(0),
              out.stride(1), num_heads, key_dim, value_dim, _stream())
    return out, (state[0] if squeeze_state else state)


@gdn_recurrent_prefill_sequential.register_fake
def _(q, k, v, beta, g, cu_seqlens=None):
    num_heads, key_dim, value_dim = q.shape[1], q.shape[2], v.shape[2]
    shape = (num_heads, key_dim, value_dim) if cu_seqlens is None else (cu_seqlens.numel() - 1, num_heads, key_dim, value_dim)
    return torch.empty_like(v), torch.empty(shape, dtype=torch.float32, device=q.device)


# =========================================================================== varlen causal prefill attention
@torch.library.custom_op("wy_lib::gqa_attention_varlen_causal", mutates_args=(), device_types="cuda")
def gqa_attention_varlen_causal(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens: torch.Tensor,
                                max_seqlen: int) -> torch.Tensor:
    """Replaces triton_kernels/gqa_attention_varlen_causal.py:214-278.  q [T,H_q,D], k/v [T,H_kv,D] bf16 packed;
    `max_seqlen` is a host int that only sizes the grid."""
    assert q.dtype == torch.bfloat16 and k.dtype == v.dtype == torch.bfloat16
    assert q.ndim == 3 and k.ndim == 3 and v.ndim == 3
    assert cu_seqlens.dtype == torch.int32 and cu_seqlens.ndim == 1
    total_tokens, num_q_head, d_model = q.shape
    assert k.shape == v.shape
    assert k.shape[0] == total_tokens and k.shape[2] == d_model
    num_kv_head = k.shape[1]
    assert num_q_head % num_kv_head == 0
    batch = cu_seqlens.numel() - 1
    assert batch >= 1
    _require_cuda(q, k, v, cu_seqlens)
    q, k, v = map(_inner_contiguous, (q, k, v))
    out = torch.empty_like(q)
    assert out.stride(2) == 1
    cu_seqlens = cu_seqlens.contiguous()  # kept alive until the launch is enqueued
    _lib.call("b200_gqa_varlen_causal", _ptr(q), q.stride(0), q.stride(1), _ptr(k), k.stride(0), k.stride(1), _ptr(v),
              v.stride(0), v.stride(1), _ptr(out), out.stride(0), out.stride(1), _ptr(cu_seqlens), batch,
              total_tokens, int(max_seqlen), num_q_head, num_kv_head, d_model, _stream())
    return out


@gqa_attention_varlen_causal.register_fake
def _(q, k, v, cu_seqlens, max_seqlen) -> torch.Tensor:
    return torch.empty_like(q)


def build_cu_seqlens(lengths, *, device="cuda"):
    """Length list -> (cu_seqlens [B+1] int32, max_seqlen).  triton_kernels/gqa_attention_varlen_causal.py:288-298."""
    cu = [0]
    for n in lengths:
        cu.append(cu[-1] + n)
    return torch.tensor(cu, dtype=torch.int32, device=device), (max(lengths) if lengths else 0)


def fused_prefill_attention(q, k, v, gate, k_cache, v_cache, block_table, cu_seqlens, position_ids, inv_freq,
                            rotary_dim, max_seqlen, out=None) -> torch.Tensor:
    """RoPE(q, k) + packed causal attention + sigmoid gate + paged KV scatter (two launches) -> [T, H_q*D] bf16.
    q [T,H_q,D], k/v [T,H_kv,D] are the post-norm, PRE-RoPE projections (any token/head strides); gate [T, H_q*D];
    position_ids [1,T] or [T] int32/int64, restarting at every sequence."""
    total, num_q_heads, head_dim = q.shape
    num_kv_heads = k.shape[1]
    assert k.shape == v.shape == (total, num_kv_heads, head_dim)
    assert gate.shape == (total, num_q_heads * head_dim)
    assert q.dtype == k.dtype == v.dtype == gate.dtype == k_cache.dtype == v_cache.dtype == torch.bfloat16
    assert k_cache.shape[1:] == (num_kv_heads, PAGE_SIZE, head_dim) and v_cache.shape == k_cache.shape
    assert cu_seqlens.dtype == torch.int32 and cu_seqlens.ndim == 1 and cu_seqlens.is_contiguous()
    batch = cu_seqlens.numel() - 1
    assert block_table.dtype == torch.int32 and block_table.shape[0] == batch and block_table.stride(1) == 1
    assert block_table.shape[1] >= (max_seqlen + PAGE_SIZE - 1) // PAGE_SIZE
    position_ids = position_ids.reshape(-1)
    assert position_ids.numel() == total and position_ids.dtype in (torch.int32, torch.int64)
    assert position_ids.is_contiguous()
    assert inv_freq.dtype == torch.float32 and inv_freq.shape == (rotary_dim // 2,) and inv_freq.is_contiguous()
    assert k_cache.stride(3) == 1 and v_cache.stride(3) == 1
    _require_cuda(q, k, v, gate, k_cache, v_cache, block_table, cu_seqlens, position_ids, inv_freq)
    q, k, v, gate = map(_inner_contiguous, (q, k, v, gate))
    if out is None:
        out = torch.empty((total, num_q_heads * head_dim), dtype=torch.bfloat16, device=q.device)
    assert out.is_contiguous() and out.shape == (total, num_q_heads * head_dim)
    k_rot = torch.empty((total, num_kv_heads, head_dim), dtype=torch.bfloat16, device=q.device)  # rotated k, packed
    _lib.call("b200_fused_prefill_attention", _ptr(q), q.stride(0), q.stride(1), _ptr(k), k.stride(0), k.stride(1),
              _ptr(v), v.stride(0), v.stride(1), _ptr(gate), gate.stride(0), _ptr(k_cache), _ptr(v_cache),
              k_cache.stride(0), k_cache.stride(1), k_cache.stride(2), v_cache.stride(0), v_cache.stride(1),
              v_cache.stride(2), _ptr(block_table), block_table.stride(0), _ptr(cu_seqlens), _ptr(position_ids),
              int(position_ids.dtype == torch.int64), _ptr(inv_freq), int(rotary_dim), _ptr(k_rot), _ptr(out), batch,
              total, int(max_seqlen), num_q_heads, num_kv_heads, head_dim, _stream())
    return out


# =========================================================================== Gated DeltaNet, chunk-64 form
@torch.library.custom_op("wy_lib::gdn_chunk_prepare_wy", mutates_args=(), device_types="cuda")
def gdn_chunk_prepare_wy(k: torch.Tensor, v: torch.Tensor, beta: torch.Tensor,
                         g: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Replaces triton_kernels/gdn_recurrent_prefill.py:703-784.  Returns (w [N,H,64,DK], u_base [N,H,64,DV],
    g_cumsum [N,H,64]) in fp32 for ONE sequence of T tokens, N = cdiv(T, 64)."""
    assert k.ndim == 3 and v.ndim == 3
    assert k.shape[:2] == v.shape[:2]
    assert beta.ndim == 2 and g.ndim == 2
    assert beta.shape == g.shape == k.shape[:2]
    assert k.dtype == torch.bfloat16 and v.dtype == torch.bfloat16
    assert beta.dtype == torch.float32 and g.dtype == torch.float32
    assert k.device == v.device == beta.device == g.device
    token_num, num_heads, key_dim = k.shape
    value_dim = v.shape[-1]
    assert token_num > 0 and num_heads > 0
    _require_cuda(k)
    k, v = _inner_contiguous(k), _inner_contiguous(v)
    num_chunks = (token_num + GDN_CHUNK - 1) // GDN_CHUNK
    w = torch.empty((num_chunks, num_heads, GDN_CHUNK, key_dim), dtype=torch.float32, device=k.device)
    u_base = torch.empty((num_chunks, num_heads, GDN_CHUNK, value_dim), dtype=torch.float32, device=k.device)
    g_cumsum = torch.empty((num_chunks, num_heads, GDN_CHUNK), dtype=torch.float32, device=k.device)
    _lib.call("b200_gdn_chunk_prepare_wy", _ptr(k), k.stride(0), k.stride(1), _ptr(v), v.stride(0), v.stride(1),
              _ptr(beta), beta.stride(0), beta.stride(1), _ptr(g), g.stride(0), g.stride(1), _ptr(w), _ptr(u_base),
              _ptr(g_cumsum), token_num, num_heads, key_dim, value_dim, _stream())
    return w, u_base, g_cumsum


@gdn_chunk_prepare_wy.register_fake
def _(k, v, beta, g):
    token_num, num_heads, key_dim = k.shape
    n = (token_num + GDN_CHUNK - 1) // GDN_CHUNK
    return (torch.empty((n, num_heads, GDN_CHUNK, key_dim), dtype=torch.float32, device=k.device),
            torch.empty((n, num_heads, GDN_CHUNK, v.shape[-1]), dtype=torch.float32, device=k.device),
            torch.empty((n, num_heads, GDN_CHUNK), dtype=torch.float32, device=k.device))


@torch.library.custom_op("wy_lib::gdn_chunk_state", mutates_args=(), device_types="cuda")
def gdn_chunk_state(k: torch.Tensor, w: torch.Tensor, u_base: torch.Tensor,
                    g_cumsum: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Replaces triton_kernels/gdn_recurrent_prefill.py:825-909.  Returns (delta [N,H,64,DV], chunk_state
    [N,H,DK,DV] = state ENTERING each chunk, final_state [H,DK,DV])."""
    assert k.ndim == 3 and k.dtype == torch.bfloat16
    assert w.ndim == 4 and u_base.ndim == 4 and g_cumsum.ndim == 3
    assert w.dtype == u_base.dtype == g_cumsum.dtype == torch.float32
    assert k.device == w.device == u_base.device == g_cumsum.device
    token_num, num_heads, key_dim = k.shape
    num_chunks, state_heads, chunk_size, state_key_dim = w.shape
    value_dim = u_base.shape[-1]
    assert token_num > 0
    assert state_heads == num_heads and state_key_dim == key_dim
    assert chunk_size == GDN_CHUNK
    assert u_base.shape == (num_chunks, num_heads, chunk_size, value_dim)
    assert g_cumsum.shape == (num_chunks, num_heads, chunk_size)
    assert num_chunks == (token_num + GDN_CHUNK - 1) // GDN_CHUNK
    _require_cuda(k)
    k, w, u_base, g_cumsum = _inner_contiguous(k), w.contiguous(), u_base.contiguous(), g_cumsum.contiguous()
    delta = torch.empty_like(u_base)
    chunk_state = torch.empty((num_chunks, num_heads, key_dim, value_dim), dtype=torch.float32, device=k.device)
    final_state = torch.empty((num_heads, key_dim, value_dim), dtype=torch.float32, device=k.device)
    _lib.call("b200_gdn_chunk_state", _ptr(k), k.stride(0), k.stride(1), _ptr(w), _ptr(u_base), _ptr(g_cumsum),
              _ptr(delta), _ptr(chunk_state), _ptr(final_state), token_num, num_heads, key_dim, value_dim, _stream())
    return delta, chunk_state, final_state


@gdn_chunk_state.register_fake
def _(k, w, u_base, g_cumsum):
    _, num_heads, key_dim = k.shape
    num_chunks, _, _, value_dim = u_base.shape
    return (torch.empty_like(u_base),
            torch.empty((num_chunks, num_heads, key_dim, value_dim), dtype=torch.float32, device=k.device),
            torch.empty((num_heads, key_dim, value_dim), dtype=torch.float32, device=k.device))


@torch.library.custom_op("wy_lib::gdn_chunk_output", mutates_args=(), device_types="cuda")
def gdn_chunk_output(q: torch.Tensor, k: torch.Tensor, delta: torch.Tensor, g_cumsum: torch.Tensor,
                     chunk_state: torch.Tensor) -> torch.Tensor:
    """Replaces triton_kernels/gdn_recurrent_prefill.py:935-1006.  Returns out [T,H,DV] bf16."""
    assert q.ndim == 3 and k.ndim == 3 and q.shape == k.shape
    assert q.dtype == torch.bfloat16 and k.dtype == torch.bfloat16
    assert delta.ndim == 4 and delta.dtype == torch.float32
    assert g_cumsum.ndim == 3 and g_cumsum.dtype == torch.float32
    assert chunk_state.ndim == 4 and chunk_state.dtype == torch.float32
    assert q.device == k.device == delta.device == g_cumsum.device == chunk_state.device
    token_num, num_heads, key_dim = q.shape
    num_chunks, delta_heads, chunk_size, value_dim = delta.shape
    assert token_num > 0 and delta_heads == num_heads
    assert chunk_size == GDN_CHUNK
    assert num_chunks == (token_num + GDN_CHUNK - 1) // GDN_CHUNK
    assert g_cumsum.shape == (num_chunks, num_heads, chunk_size)
    assert chunk_state.shape == (num_chunks, num_heads, key_dim, value_dim)
    _require_cuda(q)
    q, k = _inner_contiguous(q), _inner_contiguous(k)
    delta, g_cumsum, chunk_state = delta.contiguous(), g_cumsum.contiguous(), chunk_state.contiguous()
    out = torch.empty((token_num, num_heads, value_dim), dtype=q.dtype, device=q.device)
    _lib.call("b200_gdn_chunk_output", _ptr(q), q.stride(0), q.stride(1), _ptr(k), k.stride(0), k.stride(1), _ptr(delta),
              _ptr(g_cumsum), _ptr(chunk_state), _ptr(out), out.stride(0), out.stride(1), token_num, num_heads, key_dim,
              value_dim, _stream())
    return out


@gdn_chunk_output.register_fake
def _(q, k, delta, g_cumsum, chunk_state):
    return torch.empty((q.shape[0], q.shape[1], delta.shape[-1]), dtype=q.dtype, device=q.device)


_ONE_SEQUENCE_CU: dict = {}


# One sequence walks its chunks serially: the single kernel spends ~9 us per chunk on 16 CTAs, the three stages ~3.3 us
# per chunk in the state stage plus two chunk-parallel stages, which is the shorter way from about 16 chunks on.
CHUNKED_THREE_STAGE_FROM = 1024


def call_gdn_recurrent_prefill_chunked_triton(q, k, v, beta, g):
    """Chunk-64 prefill of ONE sequence; returns (out [T,H,DV] bf16, final_state [H,DK,DV] fp32).
    triton_kernels/gdn_recurrent_prefill.py:1026-1047 (name kept for drop-in use; no Triton is involved).  The caller
    wants only the output and the final state, so up to CHUNKED_THREE_STAGE_FROM tokens the three stages run as the
    single tcgen05 kernel with cu_seqlens = [0, T] whenever its layout rules hold (128-dim heads, 16-byte aligned
    q/k/v with strides that are multiples of 8); longer sequences, and inputs outside those rules, take the three
    reference-shaped stages (tensor-core products, HBM intermediates in one workspace) in one call."""
    token_num = q.shape[0]
    fusable = (q.shape[-1] == GDN_DIM and v.shape[-1] == GDN_DIM
               and all(t.stride(-1) == 1 and t.stride(0) % 8 == 0 and t.stride(1) % 8 == 0 and t.data_ptr() % 16 == 0
                       for t in (q, k, v)))
    key = (q.device.index, token_num)
    if key not in _ONE_SEQUENCE_CU:
        if len(_ONE_SEQUENCE_CU) > 4096:
            _ONE_SEQUENCE_CU.clear()
        _ONE_SEQUENCE_CU[key] = torch.tensor([0, token_num], dtype=torch.int32, device=q.device)
    if fusable and token_num < CHUNKED_THREE_STAGE_FROM:
        out, state = gdn_chunked_prefill_packed(q, k, v, beta, g, _ONE_SEQUENCE_CU[key])
    else:
        out, state = gdn_chunked_prefill_packed(q, k, v, beta, g, _ONE_SEQUENCE_CU[key], max_seqlen=token_num,
                                                fused=False)
    return out, state[0]


def gdn_chunked_prefill_packed(q, k, v, beta, g, cu_seqlens, max_seqlen=None, fused=True, state_out=None):
    """Chunk-64 Gated-DeltaNet prefill over a PACKED batch (chunks restart at every cu_seqlens[b], zero state at each
    sequence start).  Returns (out [T,H,DV] bf16, state [B,H,DK,DV] fp32).  The reference's chunk path is
    single-sequence only (engine/runner.py:263-267); this is its packed form, equal to
    gdn_recurrent_prefill_sequential(..., cu_seqlens) up to fp32 rounding.
    fused=True: one tcgen05 kernel, state resident in tensor memory, no workspace (q/k/v need token and head strides
    that are multiples of 8 elements).  fused=False: the three reference-shaped stages through a workspace;
    `max_seqlen` (host int) sizes their grid.  `state_out` (contiguous fp32 [B,H,DK,DV]) receives the final states in
    place of a fresh tensor, e.g. a cache's own state buffer."""
    _check_gdn(q, k, v, beta, g)
    assert cu_seqlens.dtype == torch.int32 and cu_seqlens.ndim == 1 and cu_seqlens.is_cuda
    token_num, num_heads, key_dim = q.shape
    value_dim = v.shape[-1]
    batch = cu_seqlens.numel() - 1
    q, k, v = map(_inner_contiguous, (q, k, v))
    if state_out is None:
        state = torch.empty((batch, num_heads, key_dim, value_dim), dtype=torch.float32, device=q.device)
    else:
        assert state_out.shape == (batch, num_heads, key_dim, value_dim) and state_out.dtype == torch.float32
        assert state_out.is_contiguous() and state_out.device == q.device
        state = state_out
    out = torch.empty((token_num, num_heads, value_dim), dtype=q.dtype, device=q.device)
    if fused:
        cu_seqlens = cu_seqlens.contiguous()  # kept alive until the launch is enqueued
        _lib.call("b200_gdn_chunked_prefill_fused", _ptr(q), q.stride(0), q.stride(1), _ptr(k), k.stride(0), k.stride(1),
                  _ptr(v), v.stride(0), v.stride(1), _ptr(beta), beta.stride(0), beta.stride(1), _ptr(g), g.stride(0),
                  g.stride(1), _ptr(cu_seqlens), batch, token_num, _ptr(state), _ptr(out), out.stride(0),
                  out.stride(1), num_heads, key_dim, value_dim, _stream())
        return out, state
    assert max_seqlen is not None, "the three-stage path needs max_seqlen"
    nbytes = _lib.load().b200_gdn_chunked_prefill_packed_workspace_bytes(batch, token_num, num_heads)
    workspace = torch.empty(nbytes, dtype=torch.uint8, device=q.device)
    cu_seqlens = cu_seqlens.contiguous()  # kept alive until the launch is enqueued
    _lib.call("b200_gdn_chunked_prefill_packed", _ptr(q), q.stride(0), q.stride(1), _ptr(k), k.stride(0), k.stride(1),
              _ptr(v), v.stride(0), v.stride(1), _ptr(beta), beta.stride(0), beta.stride(1), _ptr(g), g.stride(0),
              g.stride(1), _ptr(cu_seqlens), batch, token_num, int(max_seqlen), _ptr(workspace), _ptr(state),
              _ptr(out), out.stride(0), out.stride(1), num_heads, key_dim, value_dim, _stream())
    return out, state


# =========================================================================== row-wise layer operators (one launch each)
# Overlap flags (programmatic dependent launch, include/b200_attn.h): START = this kernel may begin while the kernel in
# front of it still runs; TRIGGER = the next kernel may begin early too (only when it is one of these operators called
# with START); PREFETCH = gdn_decode_fused may load its states before the kernel in front of it has finished.
OVERLAP_START, OVERLAP_TRIGGER, OVERLAP_PREFETCH = 1, 2, 4

_chain_enabled = True


def set_chain_overlap(enabled: bool) -> None:
    """Switch the chained launches of the small decode-step operators on or off, process-wide (b200_set_chain_overlap);
    on by default.  Off, every operator is launched plainly and `chain_flags()` is 0."""
    global _chain_enabled
    _chain_enabled = bool(enabled)
    _lib.call("b200_set_chain_overlap", int(_chain_enabled))


def chain_flags() -> int:
    """Overlap flags for an operator that is called as one link of a chain of this package's kernels by a caller that
    knows nothing about its neighbours (the drop-in operators): start early, let the successor start early."""
    return OVERLAP_START | OVERLAP_TRIGGER if _chain_enabled else 0


def add_rmsnorm(x, weight, eps: float, residual=None, overlap: int = 0):
    """Qwen RMSNorm `x * rsqrt(mean(x^2) + eps) * (1 + weight)` over the last dim (triton_kernels/qwen_rmsnorm.py:70-73),
    optionally fused with the residual add in front of it (triton_kernels/residual_add.py).
    x: [rows, dim] or a [n, H, dim] column view of a fused projection (last dim contiguous).  Returns norm, or
    (sum, norm) when `residual` [rows, dim] is given (sum = bf16(x + residual), the new residual stream)."""
    assert x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and weight.is_contiguous()
    _require_cuda(x, weight)
    x = _inner_contiguous(x)
    dim = x.shape[-1]
    if x.ndim == 3:
        outer, inner, count = x.stride(0), x.stride(1), x.shape[1]
        rows = x.shape[0] * x.shape[1]
    else:
        assert x.ndim == 2
        outer, inner, count, rows = x.stride(0), 0, 1, x.shape[0]
    norm = torch.empty(x.shape, dtype=torch.bfloat16, device=x.device)
    total = None
    if residual is not None:
        assert x.ndim == 2 and residual.shape == x.shape and residual.dtype == torch.bfloat16 and residual.stride(1) == 1
        total = torch.empty(x.shape, dtype=torch.bfloat16, device=x.device)
    _lib.call("b200_add_rmsnorm", _ptr(x), outer, inner, count, _ptr(residual) if residual is not None else None,
              residual.stride(0) if residual is not None else 0, _ptr(weight), _ptr(total) if total is not None else None,
              _ptr(norm), rows, dim, float(eps), int(overlap), _stream())
    return norm if residual is None else (total, norm)


def swiglu_fused(gate_up, intermediate: int, overlap: int = 0):
    """bf16(silu(gate_up[:, :I]) * gate_up[:, I:2I]) from the fused gate/up projection (triton_kernels/swiglu.py)."""
    assert gate_up.ndim == 2 and gate_up.dtype == torch.bfloat16 and gate_up.stride(1) == 1
    assert gate_up.shape[1] >= 2 * intermediate
    _require_cuda(gate_up)
    out = torch.empty((gate_up.shape[0], intermediate), dtype=torch.bfloat16, device=gate_up.device)
    _lib.call("b200_swiglu", _ptr(gate_up), gate_up.stride(0), _ptr(out), gate_up.shape[0], int(intermediate),
              int(overlap), _stream())
    return out


def gdn_decode_prep(qkv, conv_state, weight4, a, b, a_log, dt_bias, num_heads: int):
    """One decode token per sequence of a Gated-DeltaNet layer: conv state shift + depthwise conv4 + SiLU
    (triton_kernels/depthwise_causal_conv4_decode.py), q/k L2 norms and the beta / g gates
    (triton_kernels/gdn_qk_norm_gates.py:68-89) in one launch.  qkv [B, 3*H*128] (row view), conv_state [B,4,3*H*128]
    (updated in place), weight4 [4, 3*H*128], a/b [B,H] bf16 (row views).
    Returns q_n, k_n, v [B,H,128] bf16 and beta, g [B,H] fp32."""
    batch, width = qkv.shape
    assert width == 3 * num_heads * GDN_DIM and qkv.stride(1) == 1 and qkv.dtype == torch.bfloat16
    assert conv_state.shape == (batch, 4, width) and conv_state.is_contiguous() and conv_state.dtype == torch.bfloat16
    assert weight4.shape == (4, width) and weight4.is_contiguous() and weight4.dtype == torch.bfloat16
    assert a.shape == b.shape == (batch, num_heads) and a.dtype == b.dtype == torch.bfloat16
    assert a.stride(1) == 1 and b.stride(1) == 1
    assert a_log.dtype == torch.float32 and a_log.is_contiguous() and dt_bias.dtype == torch.bfloat16
    _require_cuda(qkv, conv_state, weight4, a, b, a_log, dt_bias)
    dev = qkv.device
    q_n = torch.empty((batch, num_heads, GDN_DIM), dtype=torch.bfloat16, device=dev)
    k_n, v = torch.empty_like(q_n), torch.empty_like(q_n)
    beta = torch.empty((batch, num_heads), dtype=torch.float32, device=dev)
    g = torch.empty_like(beta)
    dt_bias = dt_bias.contiguous()  # kept alive until the launch is enqueued
    _lib.call("b200_gdn_decode_prep", _ptr(qkv), qkv.stride(0), _ptr(conv_state), _ptr(weight4), _ptr(a), a.stride(0),
              _ptr(b), b.stride(0), _ptr(a_log), _ptr(dt_bias), _ptr(q_n), _ptr(k_n), _ptr(v), _ptr(beta),
              _ptr(g), batch, num_heads, GDN_DIM, _stream())
    return q_n, k_n, v, beta, g


def gdn_gated_rmsnorm_fused(x, z, weight):
    """x * rsqrt(mean(x^2) + 1e-6) * weight * silu(z) per head (triton_kernels/gdn_gated_rmsnorm.py:54-67).
    x [n,H,128] contiguous, z [n, H*128] row view, weight [128] fp32 -> [n, H*128] bf16."""
    n, heads, dim = x.shape
    assert dim == GDN_DIM and x.is_contiguous() and x.dtype == torch.bfloat16
    assert z.shape == (n, heads * dim) and z.stride(1) == 1 and z.dtype == torch.bfloat16
    assert weight.dtype == torch.float32 and weight.shape == (dim,) and weight.is_contiguous()
    _require_cuda(x, z, weight)
    out = torch.empty((n, heads * dim), dtype=torch.bfloat16, device=x.device)
    _lib.call("b200_gdn_gated_rmsnorm", _ptr(x), _ptr(z), z.stride(0), _ptr(weight), _ptr(out), n * heads, heads, dim,
              _stream())
    return out


def gdn_decode_fused(fused, conv_state, weight4, a_log, dt_bias, norm_weight, state, num_heads: int, overlap: int = 0):
    """The Gated-DeltaNet mixer of one decode token per sequence between its projections in ONE launch: conv + SiLU,
    q/k norms, gates, delta-rule step and gated RMSNorm (engine/runner.py:431-441).  fused [B, 4*H*128 + 2*H] is the
    row of the fused input projection ([q|k|v|z|a|b]); conv_state [B,4,3*H*128] and state [B,H,128,128] are updated in
    place.  Returns the normed mixer output [B, H*128] bf16 (the input of out_proj).
    overlap: OVERLAP_* flags; OVERLAP_PREFETCH lets the kernel load conv_state / state while the kernel before it in
    the stream is still running: only valid when that kernel does not write them."""
    batch = fused.shape[0]
    kd = num_heads * GDN_DIM
    assert fused.shape == (batch, 4 * kd + 2 * num_heads) and fused.stride(1) == 1 and fused.dtype == torch.bfloat16
    assert conv_state.shape == (batch, 4, 3 * kd) and conv_state.is_contiguous() and conv_state.dtype == torch.bfloat16
    assert weight4.shape == (4, 3 * kd) and weight4.is_contiguous() and weight4.dtype == torch.bfloat16
    assert a_log.dtype == torch.float32 and a_log.is_contiguous() and dt_bias.dtype == torch.bfloat16
    assert norm_weight.dtype == torch.float32 and norm_weight.shape == (GDN_DIM,) and norm_weight.is_contiguous()
    assert state.shape == (batch, num_heads, GDN_DIM, GDN_DIM) and state.is_contiguous() and state.dtype == torch.float32
    _require_cuda(fused, conv_state, weight4, a_log, dt_bias, norm_weight, state)
    out = torch.empty((batch, kd), dtype=torch.bfloat16, device=fused.device)
    dt_bias = dt_bias.contiguous()  # kept alive until the launch is enqueued
    _lib.call("b200_gdn_decode_fused", _ptr(fused), fused.stride(0), _ptr(conv_state), _ptr(weight4), _ptr(a_log),
              _ptr(dt_bias), _ptr(norm_weight), _ptr(state), _ptr(out), batch, num_heads, GDN_DIM,
              int(overlap), _stream())
    return out


def argmax_workspace(device="cuda") -> torch.Tensor:
    """Zero-filled workspace for `argmax_rows` (one per stream of calls; every call leaves it zero again)."""
    return torch.zeros(_lib.load().b200_argmax_rows_workspace_bytes(), dtype=torch.uint8, device=device)


def argmax_rows(logits, workspace, out=None, overlap: int = 0) -> torch.Tensor:
    """ids[r] = argmax_n logits[r, n] for fp32 logits [rows, n], ties to the lowest index (the arg-max half of
    triton_kernels/vocab_argmax.py:141-200; the logits come from a library GEMM).  Returns int64 [rows]."""
    assert logits.ndim == 2 and logits.dtype == torch.float32 and logits.stride(1) == 1
    _require_cuda(logits, workspace)
    rows, n = logits.shape
    if out is None:
        out = torch.empty(rows, dtype=torch.int64, device=logits.device)
    assert out.dtype == torch.int64 and out.is_contiguous() and out.numel() == rows
    _lib.call("b200_argmax_rows", _ptr(logits), logits.stride(0), _ptr(out), _ptr(workspace), rows, n, int(overlap),
              _stream())
    return out


def lm_head_argmax(hidden, table, workspace, out=None, overlap: int = 0) -> torch.Tensor:
    """ids[b] = argmax_v <hidden[b], table[v]> (fp32 accumulation, ties to the lowest id) in one launch: the tied LM head
    and greedy sampling of triton_kernels/vocab_argmax.py:141-200 without writing the logits.  hidden [M <= 32, K <= 1280]
    bf16, table [V, K] bf16 contiguous, V a multiple of 8; workspace from `argmax_workspace`.  Returns int64 [M]."""
    assert hidden.ndim == 2 and table.ndim == 2 and hidden.shape[1] == table.shape[1]
    assert hidden.dtype == table.dtype == torch.bfloat16 and table.is_contiguous() and hidden.stride(1) == 1
    _require_cuda(hidden, table, workspace)
    m, k = hidden.shape
    if out is None:
        out = torch.empty(m, dtype=torch.int64, device=hidden.device)
    assert out.dtype == torch.int64 and out.is_contiguous() and out.numel() == m
    _lib.call("b200_lm_head_argmax", _ptr(hidden), hidden.stride(0), _ptr(table), _ptr(out), _ptr(workspace), m,
              table.shape[0], k, int(overlap), _stream())
    return out


SKINNY_GEMM_MAX_M, SKINNY_GEMM_MAX_K = 32, 1280      # MAX_K: X staged whole; longer rows take the wide-K form
SKINNY_GEMM_PAIR_MAX_K = 4096                        # up to here long rows are split over a pair of CTAs (K % 256 == 0)
SKINNY_GEMM_WIDE_CHUNK, SKINNY_GEMM_WIDE_MAX_K = 1024, 16384


def skinny_gemm_supports(m: int, n: int, k: int, swiglu: bool = False) -> bool:
    """Whether `skinny_gemm` takes an [m, k] x [n, k]^T product (the shape rules of b200_skinny_gemm[_swiglu])."""
    if not (0 < m <= SKINNY_GEMM_MAX_M and n > 0 and n % 8 == 0 and k >= 128 and k % 128 == 0):
        return False
    if k <= SKINNY_GEMM_MAX_K:
        return True
    if swiglu or k > SKINNY_GEMM_WIDE_MAX_K:
        return False
    chunks = -(-k // SKINNY_GEMM_WIDE_CHUNK)
    return k % (chunks * 128) == 0


def skinny_gemm(x, weight, overlap: int = 0, swiglu: bool = False):
    """y = x @ weight^T for a decode batch (x [M <= 32, K] bf16, weight [N, K] bf16 contiguous), the weight streamed
    once from HBM (triton_kernels/gemm_2d.py for the decode-step projections).  K <= 1280: every warp owns 16 outputs
    and the whole K; longer rows (the out / o / down projections): 16 outputs per step, K split over the warps of a
    pair of CTAs (K <= 4096) or of one CTA with X staged in chunks (`skinny_gemm_supports` tells which shapes are taken).
    swiglu=True: weight = [gate rows | up rows] [2*I, K] and the result is silu(bf16(x.gate_j)) * bf16(x.up_j), [M, I]
    (the fused gate/up projection followed by triton_kernels/swiglu.py, one launch)."""
    assert x.ndim == 2 and weight.ndim == 2 and x.shape[1] == weight.shape[1]
    assert x.dtype == weight.dtype == torch.bfloat16 and weight.is_contiguous() and x.stride(1) == 1
    m, k = x.shape
    n = weight.shape[0]
    if swiglu:
        assert n % 2 == 0
        n //= 2
    _require_cuda(x, weight)
    y = torch.empty((m, n), dtype=torch.bfloat16, device=x.device)
    _lib.call("b200_skinny_gemm_swiglu" if swiglu else "b200_skinny_gemm", _ptr(x), x.stride(0), _ptr(weight), _ptr(y),
              y.stride(0), m, n, k, int(overlap), _stream())
    return y


# eager callers reach the implementations directly; the registered operators stay available as `<name>.op` and under
# torch.ops.wy_lib (see _direct.py)
from ._direct import rebind as _rebind  # noqa: E402

_rebind(globals())
