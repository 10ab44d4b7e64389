"""The reference's operators AROUND the attention / Gated-DeltaNet path, registered under their `wy_lib::*` names
with the reference's schemas so that `engine/runner.py` and `engine/cache.py` run unchanged (eager or under
`torch.compile`, hence a fake implementation per operator).

Each one launches a CUDA kernel of libb200attn.so where the library has one for the shape (all the model's shapes);
projections of more than 32 rows go to cuBLAS through `torch.nn.functional.linear`, and a shape outside a kernel's
rules runs the PyTorch restatement of `glue.py` on the same device.  Nothing runs on the CPU.

Also here: the two reference operators that `engine/runner.py` imports for its single-sequence baselines, served by the
path kernels - fixed-length causal attention by the packed varlen kernel with `cu_seqlens = [0, T]`, the contiguous
B=1 decode cache by the paged kernels over an identity page table.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import _lib, glue, ops
from .ops import _ptr, _require_cuda, _stream

CONV_KERNEL_SIZE = 4   # triton_kernels/depthwise_causal_conv4_decode.py:66


def _aligned16(*tensors) -> bool:
    return all(t.data_ptr() % 16 == 0 for t in tensors)


# =========================================================================== projections
@torch.library.custom_op("wy_lib::gemm_2d", mutates_args=(), device_types="cuda")
def gemm_2d(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """y = x @ weight^T, bf16 in / out, fp32 accumulation.  Replaces triton_kernels/gemm_2d.py:188-226.
    Decode batches (M <= 32) stream the weight once through `b200_skinny_gemm`; larger M is a library GEMM."""
    assert x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
    assert x.shape[1] == weight.shape[1]
    assert x.shape[1] % 128 == 0
    _require_cuda(x, weight)
    m, k = x.shape
    n = weight.shape[0]
    if (ops.skinny_gemm_supports(m, n, k) and k <= ops.SKINNY_GEMM_PAIR_MAX_K and weight.is_contiguous()
            and x.stride(1) == 1 and x.stride(0) % 8 == 0 and _aligned16(x, weight)):
        return ops.skinny_gemm(x, weight, overlap=ops.chain_flags())
    return F.linear(x, weight)


@gemm_2d.register_fake
def _(x, weight):
    return torch.empty((x.shape[0], weight.shape[0]), dtype=x.dtype, device=x.device)


_ARGMAX_WS: dict = {}


def _argmax_workspace(device) -> torch.Tensor:
    key = torch.device(device).index
    if key not in _ARGMAX_WS:
        _ARGMAX_WS[key] = ops.argmax_workspace(device)
    return _ARGMAX_WS[key]


@torch.library.custom_op("wy_lib::lm_head_argmax", mutates_args=(), device_types="cuda")
def lm_head_argmax(hidden: torch.Tensor, weight: torch.Tensor, last_only: bool = True) -> torch.Tensor:
    """Tied LM head + greedy arg-max without materialising the logits; ties go to the lowest id.
    Replaces triton_kernels/vocab_argmax.py:135-223.  last_only=True: the last row of `hidden` only, returns a 0-d
    int64 tensor; False: one id per row, int64 [rows].  The first call on a device allocates a small workspace (make it
    outside CUDA-graph capture, as the reference runner's warm-up steps do)."""
    assert hidden.ndim == 2 and weight.ndim == 2
    assert hidden.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
    assert hidden.device == weight.device
    assert hidden.is_contiguous() and weight.is_contiguous()
    token_num, hidden_size = hidden.shape
    vocab_size, weight_hidden_size = weight.shape
    assert token_num > 0 and vocab_size > 0
    assert weight_hidden_size == hidden_size
    assert hidden_size % 128 == 0
    _require_cuda(hidden, weight)
    rows = hidden[token_num - 1:] if last_only else hidden
    if hidden_size <= ops.SKINNY_GEMM_MAX_K and vocab_size % 8 == 0 and _aligned16(rows, weight):
        ws = _argmax_workspace(hidden.device)
        ids = torch.empty(rows.shape[0], dtype=torch.int64, device=hidden.device)
        for r0 in range(0, rows.shape[0], ops.SKINNY_GEMM_MAX_M):
            r1 = min(r0 + ops.SKINNY_GEMM_MAX_M, rows.shape[0])
            ops.lm_head_argmax(rows[r0:r1], weight, ws, out=ids[r0:r1], overlap=ops.chain_flags())
    else:
        ids = glue.lm_head_argmax(rows, weight, last_only=False)
    return ids[0].clone() if last_only else ids


@lm_head_argmax.register_fake
def _(hidden, weight, last_only=True):
    shape = () if last_only else (hidden.shape[0],)
    return torch.empty(shape, dtype=torch.int64, device=hidden.device)


# =========================================================================== norms / element-wise
@torch.library.custom_op("wy_lib::qwen_rmsnorm", mutates_args=(), device_types="cuda")
def qwen_rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """x * rsqrt(mean(x^2) + eps) * (1 + weight) over the last dim; x is [rows, D] contiguous or a [B, H, D] view with
    uniform strides (a column slice of a fused projection).  Replaces triton_kernels/qwen_rmsnorm.py:98-146."""
    assert x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
    assert weight.is_contiguous()
    assert x.stride(-1) == 1
    d_model = x.shape[-1]
    assert weight.shape == (d_model,)
    assert x.ndim in (2, 3)
    if x.ndim == 2:
        assert x.is_contiguous(), "a 2-D input is read as flat rows and must be contiguous"
    _require_cuda(x, weight)
    strides_ok = all(s % 8 == 0 for s in x.stride()[:-1])
    if d_model % 256 == 0 and d_model <= 8192 and strides_ok and _aligned16(x, weight):
        return ops.add_rmsnorm(x, weight, eps, overlap=ops.chain_flags())
    return glue.qwen_rmsnorm(x, weight, eps).contiguous()


@qwen_rmsnorm.register_fake
def _(x, weight, eps=1e-6):
    return torch.empty(x.shape, dtype=x.dtype, device=x.device)


@torch.library.custom_op("wy_lib::residual_add", mutates_args=(), device_types="cuda")
def residual_add(x: torch.Tensor, residual: torch.Tensor) -> torch.Tensor:
    """bf16(x + residual).  Replaces triton_kernels/residual_add.py:23-50."""
    assert x.shape == residual.shape
    assert x.dtype == torch.bfloat16 and residual.dtype == torch.bfloat16
    assert x.device == residual.device
    assert x.is_contiguous() and residual.is_contiguous()
    assert x.numel() > 0
    _require_cuda(x, residual)
    out = torch.empty_like(x)
    if _aligned16(x, residual, out):
        _lib.call("b200_residual_add", _ptr(x), _ptr(residual), _ptr(out), x.numel(), _stream())
        return out
    return x + residual


@residual_add.register_fake
def _(x, residual):
    return torch.empty_like(x)


@torch.library.custom_op("wy_lib::swiglu", mutates_args=(), device_types="cuda")
def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """bf16(silu(gate) * up); gate / up may be column views of one fused projection.
    Replaces triton_kernels/swiglu.py:75-110."""
    assert gate.ndim == 2 and up.ndim == 2
    assert gate.shape == up.shape
    assert gate.dtype == torch.bfloat16 and up.dtype == torch.bfloat16
    assert gate.device == up.device
    num_rows, num_cols = gate.shape
    assert num_rows > 0 and num_cols > 0
    _require_cuda(gate, up)
    out = torch.empty((num_rows, num_cols), dtype=gate.dtype, device=gate.device)
    if (num_cols % 8 == 0 and gate.stride(1) == 1 and up.stride(1) == 1 and gate.stride(0) % 8 == 0
            and up.stride(0) % 8 == 0 and _aligned16(gate, up, out)):
        _lib.call("b200_swiglu_pair", _ptr(gate), gate.stride(0), _ptr(up), up.stride(0), _ptr(out), num_rows, num_cols,
                  _stream())
        return out
    return glue.swiglu(gate, up).contiguous()


@swiglu.register_fake
def _(gate, up):
    return torch.empty(gate.shape, dtype=gate.dtype, device=gate.device)


@torch.library.custom_op("wy_lib::embedding_gather", mutates_args=(), device_types="cuda")
def embedding_gather(input_ids: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """Rows of the embedding table.  Replaces triton_kernels/embedding_gather.py:62-100."""
    assert input_ids.ndim == 1
    assert input_ids.dtype in (torch.int32, torch.int64)
    assert input_ids.is_contiguous()
    assert weight.ndim == 2 and weight.dtype == torch.bfloat16
    assert weight.is_contiguous()
    assert input_ids.device == weight.device
    token_num, d_model = input_ids.shape[0], weight.shape[1]
    assert token_num > 0 and weight.shape[0] > 0
    _require_cuda(input_ids, weight)
    out = torch.empty((token_num, d_model), dtype=weight.dtype, device=weight.device)
    if d_model % 8 == 0 and _aligned16(weight, out):
        _lib.call("b200_embedding_gather", _ptr(input_ids), int(input_ids.dtype == torch.int64), _ptr(weight), _ptr(out),
                  token_num, d_model, _stream())
        return out
    return glue.embedding_gather(input_ids, weight)


@embedding_gather.register_fake
def _(input_ids, weight):
    return torch.empty((input_ids.shape[0], weight.shape[1]), dtype=weight.dtype, device=weight.device)


# =========================================================================== Gated-DeltaNet input pipeline
@torch.library.custom_op("wy_lib::depthwise_causal_conv4_prefill", mutates_args=(), device_types="cuda")
def depthwise_causal_conv4_prefill(x: torch.Tensor, weight: torch.Tensor,
                                   seq_start: torch.Tensor | None = None) -> torch.Tensor:
    """Depthwise causal conv (4 taps) + SiLU over a packed buffer; with `seq_start` [T] int32 no tap reaches before
    the first row of its own sequence.  Replaces triton_kernels/depthwise_causal_conv4_prefill.py:108-170."""
    assert x.ndim == 2
    assert weight.ndim in (2, 3)
    assert x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
    assert x.device == weight.device
    token_num, hidden_dim = x.shape
    assert token_num > 0 and hidden_dim > 0
    if weight.ndim == 2:
        assert weight.shape == (hidden_dim, 4)
        w_d, w_k = weight.stride(0), weight.stride(1)
    else:
        assert weight.shape == (hidden_dim, 1, 4)
        w_d, w_k = weight.stride(0), weight.stride(2)
    if seq_start is not None:
        assert seq_start.shape == (token_num,) and seq_start.dtype == torch.int32
        assert seq_start.device == x.device
        seq_start = seq_start.contiguous()
    _require_cuda(x, weight)
    out = torch.empty((token_num, hidden_dim), dtype=x.dtype, device=x.device)
    if hidden_dim % 8 == 0 and x.stride(1) == 1 and x.stride(0) % 8 == 0 and _aligned16(x, out):
        _lib.call("b200_conv4_prefill", _ptr(x), x.stride(0), _ptr(weight), w_d, w_k, _ptr(seq_start), _ptr(out),
                  out.stride(0), token_num, hidden_dim, _stream())
        return out
    return glue.depthwise_causal_conv4_prefill(x, weight.reshape(hidden_dim, 4), seq_start).contiguous()


@depthwise_causal_conv4_prefill.register_fake
def _(x, weight, seq_start=None):
    return torch.empty(x.shape, dtype=x.dtype, device=x.device)


@torch.library.custom_op("wy_lib::depthwise_causal_conv4_decode", mutates_args=("state",), device_types="cuda")
def depthwise_causal_conv4_decode(x: torch.Tensor, state: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """One token per sequence: `state` [B,4,D] (the conv INPUT history) shifts up a row in place, x becomes its last
    row, y = silu(sum_r weight[r] * state[:, r]).  weight is the contiguous [4, D] decode layout.
    Replaces triton_kernels/depthwise_causal_conv4_decode.py:152-207."""
    assert x.ndim == 2, "decode takes one token per sequence: x is [B, D]"
    assert state.ndim == 3 and weight.ndim == 2
    assert x.dtype == torch.bfloat16 and state.dtype == torch.bfloat16
    assert weight.dtype == torch.bfloat16
    assert x.device == state.device == weight.device
    batch, hidden_dim = x.shape
    assert state.shape == (batch, CONV_KERNEL_SIZE, hidden_dim), (
        f"state must be [B,4,D]={(batch, CONV_KERNEL_SIZE, hidden_dim)}, got {tuple(state.shape)}")
    assert weight.shape == (CONV_KERNEL_SIZE, hidden_dim), (
        f"weight must be [4,D]={(CONV_KERNEL_SIZE, hidden_dim)}, got {tuple(weight.shape)}; "
        "convert the checkpoint's [D,1,4] with conv_weight_for_decode()")
    assert state.is_contiguous() and weight.is_contiguous(), (
        "state / weight must be contiguous [B,4,D] / [4,D], not a transposed view of [D,4]")
    _require_cuda(x, state, weight)
    out = torch.empty((batch, hidden_dim), dtype=x.dtype, device=x.device)
    if hidden_dim % 8 == 0 and x.stride(1) == 1 and x.stride(0) % 8 == 0 and _aligned16(x, state, weight, out):
        _lib.call("b200_conv4_decode", _ptr(x), x.stride(0), _ptr(state), _ptr(weight), _ptr(out), out.stride(0), batch,
                  hidden_dim, _stream())
        return out
    return glue.depthwise_causal_conv4_decode(x, state, weight).contiguous()


@depthwise_causal_conv4_decode.register_fake
def _(x, state, weight):
    return torch.empty(x.shape, dtype=x.dtype, device=x.device)


def conv_state_from_prefill(x: torch.Tensor) -> torch.Tensor:
    """Conv input [T, D] of ONE sequence -> its initial decode state [4, D]: the last 4 rows, zero rows on top when
    T < 4.  triton_kernels/depthwise_causal_conv4_decode.py:227-240."""
    token_num, hidden_dim = x.shape
    state = torch.zeros((CONV_KERNEL_SIZE, hidden_dim), dtype=x.dtype, device=x.device)
    take = min(token_num, CONV_KERNEL_SIZE)
    state[CONV_KERNEL_SIZE - take:] = x[-take:]
    return state


@torch.library.custom_op("wy_lib::conv_state_from_packed_prefill", mutates_args=("state",), device_types="cuda")
def conv_state_from_packed_prefill(state: torch.Tensor, x: torch.Tensor, cu_seqlens: torch.Tensor) -> None:
    """state[b] = the last 4 conv-input rows of sequence b of the packed buffer x (zero rows on top of short
    sequences), written in place.  Replaces triton_kernels/depthwise_causal_conv4_decode.py:332-374."""
    total_tokens, hidden_dim = x.shape
    batch = cu_seqlens.shape[0] - 1
    assert state.shape == (batch, CONV_KERNEL_SIZE, hidden_dim), (
        f"state shape {tuple(state.shape)} does not match (B={batch}, K={CONV_KERNEL_SIZE}, D={hidden_dim})")
    assert state.dtype == x.dtype
    assert cu_seqlens.dtype == torch.int32 and cu_seqlens.ndim == 1
    assert x.stride(1) == 1, "the channel dim of x must be contiguous"
    _require_cuda(state, x, cu_seqlens)
    if (x.dtype == torch.bfloat16 and state.is_contiguous() and hidden_dim % 8 == 0 and x.stride(0) % 8 == 0
            and _aligned16(x, state)):
        _lib.call("b200_conv_state_from_packed_prefill", _ptr(state), _ptr(x), x.stride(0), _ptr(cu_seqlens.contiguous()),
                  batch, hidden_dim, _stream())
    else:
        glue.conv_state_from_packed_prefill(state, x, cu_seqlens)


@conv_state_from_packed_prefill.register_fake
def _(state, x, cu_seqlens) -> None:
    return None


def conv_weight_for_decode(weight: torch.Tensor) -> torch.Tensor:
    """Checkpoint layout [D,1,4] or [D,4] -> the contiguous [4, D] the decode operator reads.
    triton_kernels/depthwise_causal_conv4_decode.py:382-391."""
    if weight.ndim == 3:
        weight = weight.squeeze(1)
    assert weight.ndim == 2 and weight.shape[1] == CONV_KERNEL_SIZE
    return weight.transpose(0, 1).contiguous()


@torch.library.custom_op("wy_lib::gdn_qk_norm_gates", mutates_args=(), device_types="cuda")
def gdn_qk_norm_gates(q: torch.Tensor, k: torch.Tensor, a: torch.Tensor, b: torch.Tensor, a_log: torch.Tensor,
                      dt_bias: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """q_n = l2norm(q) * D^-0.5, k_n = l2norm(k) (bf16), beta = sigmoid(b), g = -exp(a_log) * softplus(a + dt_bias)
    (fp32).  Replaces triton_kernels/gdn_qk_norm_gates.py:128-200."""
    assert q.ndim == 3 and k.ndim == 3
    assert q.shape == k.shape
    assert a.ndim == 2 and b.ndim == 2 and a.shape == b.shape
    assert a_log.ndim == 1 and dt_bias.ndim == 1
    assert q.dtype == torch.bfloat16 and k.dtype == torch.bfloat16
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
    assert a_log.dtype == torch.float32 and dt_bias.dtype == torch.bfloat16
    assert q.device == k.device == a.device == b.device == a_log.device == dt_bias.device
    token_num, num_heads, head_dim = q.shape
    assert token_num > 0
    assert a.shape == (token_num, num_heads)
    assert a_log.shape == (num_heads,) and dt_bias.shape == (num_heads,)
    _require_cuda(q)
    ok = (head_dim == ops.GDN_DIM and q.stride(2) == 1 and k.stride(2) == 1 and a.stride(1) == 1 and b.stride(1) == 1
          and all(s % 4 == 0 for s in (q.stride(0), q.stride(1), k.stride(0), k.stride(1)))
          and q.data_ptr() % 8 == 0 and k.data_ptr() % 8 == 0)
    if not ok:
        q_n, k_n, beta, g = glue.gdn_qk_norm_gates(q, k, a, b, a_log, dt_bias)
        return q_n.contiguous(), k_n.contiguous(), beta.contiguous(), g.contiguous()
    q_n = torch.empty((token_num, num_heads, head_dim), dtype=q.dtype, device=q.device)
    k_n = torch.empty_like(q_n)
    beta = torch.empty((token_num, num_heads), dtype=torch.float32, device=q.device)
    g = torch.empty_like(beta)
    a_log, dt_bias = a_log.contiguous(), dt_bias.contiguous()
    _lib.call("b200_gdn_qk_norm_gates", _ptr(q), q.stride(0), q.stride(1), _ptr(k), k.stride(0), k.stride(1), _ptr(a),
              a.stride(0), _ptr(b), b.stride(0), _ptr(a_log), _ptr(dt_bias), _ptr(q_n), _ptr(k_n), _ptr(beta), _ptr(g),
              token_num, num_heads, head_dim, _stream())
    return q_n, k_n, beta, g


@gdn_qk_norm_gates.register_fake
def _(q, k, a, b, a_log, dt_bias):
    q_n = torch.empty(q.shape, dtype=q.dtype, device=q.device)
    beta = torch.empty(q.shape[:2], dtype=torch.float32, device=q.device)
    return q_n, torch.empty_like(q_n), beta, torch.empty_like(beta)


@torch.library.custom_op("wy_lib::gdn_gated_rmsnorm", mutates_args=(), device_types="cuda")
def gdn_gated_rmsnorm(x: torch.Tensor, z: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """x * rsqrt(mean(x^2) + 1e-6) * weight * silu(z) per head, [T, H, D] bf16.
    Replaces triton_kernels/gdn_gated_rmsnorm.py:95-140."""
    assert x.ndim == 3 and z.ndim == 3
    assert x.shape == z.shape
    assert x.dtype == torch.bfloat16 and z.dtype == torch.bfloat16
    assert weight.ndim == 1 and weight.dtype == torch.float32
    assert x.device == z.device == weight.device
    token_num, head_num, d_model = x.shape
    assert token_num > 0
    assert weight.shape == (d_model,)
    _require_cuda(x, z, weight)
    if (d_model == ops.GDN_DIM and x.is_contiguous() and z.stride(2) == 1 and z.stride(1) == d_model
            and z.stride(0) % 4 == 0 and z.data_ptr() % 8 == 0 and weight.is_contiguous()):
        z_rows = z.as_strided((token_num, head_num * d_model), (z.stride(0), 1))
        return ops.gdn_gated_rmsnorm_fused(x, z_rows, weight).view(token_num, head_num, d_model)
    return glue.gdn_gated_rmsnorm(x, z, weight).contiguous()


@gdn_gated_rmsnorm.register_fake
def _(x, z, weight):
    return torch.empty(x.shape, dtype=x.dtype, device=x.device)


# =========================================================================== single-sequence baselines of the runner
@torch.library.custom_op("wy_lib::gqa_attention_without_kvcache_casual", mutates_args=(), device_types="cuda")
def gqa_attention_without_kvcache_casual(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """Fixed-length causal GQA prefill, q [B,H_q,T,D], k/v [B,H_kv,T,D] (any strides, unit stride on D) -> [B,H_q,T,D].
    Replaces triton_kernels/gqa_attention_without_kvcache_casual.py:148-195; served per batch row by the packed varlen
    kernel (`b200_gqa_varlen_causal`) with cu_seqlens = [0, T]."""
    assert q.dtype == torch.bfloat16 and k.dtype == torch.bfloat16 and v.dtype == torch.bfloat16
    batch_size, num_q_head, seq_len_q, d_model = q.shape
    assert k.shape == v.shape and k.shape[0] == batch_size and k.shape[3] == d_model
    assert k.shape[2] == seq_len_q, "prefill without a cache: as many keys as queries"
    num_kv_head = k.shape[1]
    assert num_q_head % num_kv_head == 0
    _require_cuda(q, k, v)
    out = torch.empty_like(q)
    if out.stride(3) != 1:
        out = torch.empty(q.shape, dtype=q.dtype, device=q.device)
    cu = _single_sequence_cu(seq_len_q, q.device)
    q, k, v = (t if t.stride(3) == 1 else t.contiguous() for t in (q, k, v))
    for row in range(batch_size):
        qr, kr, vr, orow = q[row], k[row], v[row], out[row]          # [H, T, D] views
        _lib.call("b200_gqa_varlen_causal", _ptr(qr), qr.stride(1), qr.stride(0), _ptr(kr), kr.stride(1), kr.stride(0),
                  _ptr(vr), vr.stride(1), vr.stride(0), _ptr(orow), orow.stride(1), orow.stride(0), _ptr(cu), 1,
                  seq_len_q, seq_len_q, num_q_head, num_kv_head, d_model, _stream())
    return out


@gqa_attention_without_kvcache_casual.register_fake
def _(q, k, v):
    return torch.empty_like(q)


_CU_CACHE: dict = {}


def _single_sequence_cu(token_num: int, device) -> torch.Tensor:
    """cu_seqlens = [0, T] on the device, remembered per (device, T): prompts come in few distinct lengths and the
    tensor must outlive the asynchronous launch that reads it."""
    key = (torch.device(device).index, int(token_num))
    if key not in _CU_CACHE:
        if len(_CU_CACHE) > 4096:
            _CU_CACHE.clear()
        _CU_CACHE[key] = torch.tensor([0, int(token_num)], dtype=torch.int32, device=device)
    return _CU_CACHE[key]


def allocate_kv_cache(num_kv_heads: int, max_len: int, head_dim: int, device="cuda"):
    """Contiguous single-sequence K/V cache `[H_kv, max_len, D]` bf16 (triton_kernels/gqa_attention_decode.py:504-518).
    The storage is rounded up to whole 16-token pages so that the paged kernels can read it page by page."""
    padded = (max_len + ops.PAGE_SIZE - 1) // ops.PAGE_SIZE * ops.PAGE_SIZE
    shape = (num_kv_heads, padded, head_dim)
    return (torch.zeros(shape, dtype=torch.bfloat16, device=device)[:, :max_len],
            torch.zeros(shape, dtype=torch.bfloat16, device=device)[:, :max_len])


def kv_cache_from_prefill(k: torch.Tensor, v: torch.Tensor, max_len: int):
    """Post-RoPE prefill K/V `[H_kv, T, D]` -> a preallocated cache.  triton_kernels/gqa_attention_decode.py:521-538."""
    num_kv_heads, token_num, head_dim = k.shape
    assert v.shape == k.shape
    assert token_num <= max_len
    k_cache, v_cache = allocate_kv_cache(num_kv_heads, max_len, head_dim, device=k.device)
    k_cache[:, :token_num, :] = k
    v_cache[:, :token_num, :] = v
    return k_cache, v_cache


def allocate_position(device="cuda") -> torch.Tensor:
    """Device-resident position of the single sequence, int64 [1] (triton_kernels/gqa_attention_decode.py:470-489)."""
    return torch.zeros(1, dtype=torch.int64, device=device)


def allocate_contiguous_split_scratch(num_q_heads: int, head_dim: int, device="cuda"):
    """(m, l, acc) scratch of the single-sequence split-K decode (triton_kernels/gqa_attention_decode.py:912-924)."""
    f32 = dict(dtype=torch.float32, device=device)
    return (torch.zeros((num_q_heads, ops.MAX_SPLITS), **f32), torch.zeros((num_q_heads, ops.MAX_SPLITS), **f32),
            torch.zeros((num_q_heads, ops.MAX_SPLITS, head_dim), **f32))


_IDENTITY_TABLES: dict = {}


def _paged_view(cache: torch.Tensor) -> torch.Tensor:
    """A `[H_kv, T_max, D]` cache seen as `[pages, H_kv, 16, D]` without copying: page p of head h starts at token
    16*p of that head.  The last page may reach past T_max; the storage must then extend that far (caches made by
    `allocate_kv_cache` do), because the kernels fetch whole pages and mask the rows past the sequence end."""
    heads, max_len, dim = cache.shape
    assert cache.stride(2) == 1 and cache.stride(1) == dim, "token rows of the cache must be dense"
    pages = (max_len + ops.PAGE_SIZE - 1) // ops.PAGE_SIZE
    need = cache.storage_offset() + (heads - 1) * cache.stride(0) + pages * ops.PAGE_SIZE * dim
    have = cache.untyped_storage().nbytes() // cache.element_size()
    assert need <= have, (
        f"a contiguous KV cache of {max_len} tokens is read in {pages} whole 16-token pages; its storage ends "
        "inside the last page - allocate it with allocate_kv_cache() or make max_len a multiple of 16")
    return cache.as_strided((pages, heads, ops.PAGE_SIZE, dim), (ops.PAGE_SIZE * dim, cache.stride(0), dim, 1))


def call_gqa_attention_decode_split_triton(q, k_new, v_new, k_cache, v_cache, past_len, scratch=None):
    """Single-sequence decode over a contiguous cache: append (k_new, v_new) at `past_len`, attend over past_len + 1
    tokens, return [H_q, D] bf16.  triton_kernels/gqa_attention_decode.py:927-950 (the name is kept for drop-in use;
    no Triton is involved).  q [H_q,D], k_new/v_new [H_kv,D], caches [H_kv,T_max,D], past_len an int or an int64 [1]
    device tensor; scratch = (m [H_q,128], l [H_q,128], acc [H_q,128,D]) fp32 or None.
    Served by the paged operators over an identity page table (page p = tokens 16p .. 16p+15)."""
    num_q_heads, head_dim = q.shape
    if scratch is None:
        scratch = allocate_contiguous_split_scratch(num_q_heads, head_dim, device=q.device)
    m_partial, l_partial, acc_partial = scratch
    if isinstance(past_len, int):
        pos = torch.tensor([past_len], dtype=torch.int64, device=q.device)
    else:
        pos = past_len
    assert pos.dtype == torch.int64 and pos.numel() == 1
    kc, vc = _paged_view(k_cache), _paged_view(v_cache)
    key = (q.device.index, kc.shape[0])
    if key not in _IDENTITY_TABLES:
        _IDENTITY_TABLES[key] = torch.arange(kc.shape[0], dtype=torch.int32, device=q.device).view(1, -1)
    table = _IDENTITY_TABLES[key]
    out = ops.call_paged_gqa_attention_decode_triton(
        q.unsqueeze(0), k_new.unsqueeze(0), v_new.unsqueeze(0), kc, vc, table, pos.view(1),
        (m_partial.unsqueeze(0), l_partial.unsqueeze(0), acc_partial.unsqueeze(0)))
    return out[0]


# eager callers reach the implementations directly; the registered operators stay available as `<name>.op` and under
# torch.ops.wy_lib (see _direct.py)
from ._direct import rebind as _rebind  # noqa: E402

_rebind(globals())
