"""The reference's operators that are NOT on the attention / Gated-DeltaNet path, as plain PyTorch (cuBLAS GEMMs and
built-in elementwise kernels), under the reference's own names.  They exist so that the whole model can be stepped and
timed around the CUDA operators of this package; none of them is a product kernel.  Rounding points follow the
reference kernels cited in each docstring (fp32 math, one rounding to bf16 at the end).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def gemm_2d(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """y = x @ weight^T, bf16 in / bf16 out, fp32 accumulation (triton_kernels/gemm_2d.py; weight is [N, K])."""
    return F.linear(x, weight)


def qwen_rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """x * rsqrt(mean(x^2) + eps) * (1 + weight) over the last dim (triton_kernels/qwen_rmsnorm.py:70-73)."""
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * (1.0 + weight.float())).to(x.dtype)


def residual_add(x: torch.Tensor, residual: torch.Tensor) -> torch.Tensor:
    """bf16(x.f32 + residual.f32) (triton_kernels/residual_add.py)."""
    return x + residual


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """bf16(silu(gate.f32) * up.f32) (triton_kernels/swiglu.py); accepts column views of the fused projection."""
    return (F.silu(gate.float()) * up.float()).to(gate.dtype)


def embedding_gather(token_ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """Rows of the embedding table (triton_kernels/embedding_gather.py)."""
    return table.index_select(0, token_ids.reshape(-1).long())


def lm_head_argmax(hidden: torch.Tensor, table: torch.Tensor, last_only: bool = True, argmax=None) -> torch.Tensor:
    """argmax_v <hidden, table[v]> with the tied embedding as the LM head; ties go to the lowest index
    (triton_kernels/vocab_argmax.py:141-200).  last_only=True: only the last row of hidden, returns a 0-d tensor
    (prefill of one sequence); last_only=False: one id per row, int64 [B] (batched decode).
    argmax: optional callable taking the fp32 logits [rows, V] and returning int64 [rows] (default torch.argmax)."""
    if last_only:
        hidden = hidden[-1:]
    try:
        logits = torch.mm(hidden, table.t(), out_dtype=torch.float32)    # fp32 logits straight from the GEMM
    except (TypeError, RuntimeError):
        logits = F.linear(hidden, table).float()
    ids = torch.argmax(logits, dim=-1) if argmax is None else argmax(logits)
    return ids[0] if last_only else ids


def depthwise_causal_conv4_prefill(x: torch.Tensor, weight: torch.Tensor,
                                   seq_start: torch.Tensor | None = None) -> torch.Tensor:
    """y[t,c] = silu(sum_{r=0..3} w[c,r] x[t+r-3,c]) over a packed buffer; taps that would reach before seq_start[t]
    (the first token of t's own sequence) read zero (triton_kernels/depthwise_causal_conv4_prefill.py:18-91, :108-123).
    x [T,C] bf16 (any row stride), weight [C,4] bf16, seq_start [T] int32 or None (one sequence starting at 0)."""
    total = x.shape[0]
    pos_in_seq = torch.arange(total, device=x.device)
    if seq_start is not None:
        pos_in_seq = pos_in_seq - seq_start.to(pos_in_seq.dtype)
    xf = x.float()
    wf = weight.float()
    acc = xf * wf[:, 3]
    for shift in (1, 2, 3):
        shifted = F.pad(xf, (0, 0, shift, 0))[:total]
        acc = acc + torch.where((pos_in_seq >= shift).unsqueeze(1), shifted, torch.zeros_like(shifted)) * wf[:, 3 - shift]
    return F.silu(acc).to(x.dtype)


def conv_state_from_packed_prefill(conv_state: torch.Tensor, x: torch.Tensor, cu_seqlens: torch.Tensor) -> None:
    """conv_state[b] = the last 4 rows of the conv INPUT of sequence b, zero rows in front when it is shorter
    (triton_kernels/depthwise_causal_conv4_decode.py: conv_state_from_packed_prefill).  conv_state [B,4,C]."""
    starts, ends = cu_seqlens[:-1].long(), cu_seqlens[1:].long()
    idx = ends.unsqueeze(1) - 4 + torch.arange(4, device=x.device).unsqueeze(0)       # [B,4]
    ok = idx >= starts.unsqueeze(1)
    rows = x.index_select(0, idx.clamp_min(0).reshape(-1)).view(idx.shape[0], 4, -1)
    conv_state.copy_(torch.where(ok.unsqueeze(-1), rows, torch.zeros_like(rows)))


def depthwise_causal_conv4_decode(x: torch.Tensor, conv_state: torch.Tensor, weight4: torch.Tensor) -> torch.Tensor:
    """One token per sequence: shift the state left, append x, y = silu(sum_r w[r,c] state[r,c])
    (triton_kernels/depthwise_causal_conv4_decode.py).  x [B,C], conv_state [B,4,C] (updated in place), weight4 [4,C]."""
    conv_state.copy_(torch.cat((conv_state[:, 1:], x.unsqueeze(1)), dim=1))
    acc = (conv_state.float() * weight4.float().unsqueeze(0)).sum(1)
    return F.silu(acc).to(x.dtype)


def gdn_qk_norm_gates(q, k, a, b, a_log, dt_bias):
    """q_n = q * rsqrt(sum q^2 + 1e-6) * DK^-0.5, k_n = k * rsqrt(sum k^2 + 1e-6) (both rounded to bf16);
    beta = sigmoid(b) and g = -exp(a_log) * softplus(a + dt_bias) in fp32 (triton_kernels/gdn_qk_norm_gates.py:68-89)."""
    qf, kf = q.float(), k.float()
    q_n = (qf * torch.rsqrt(qf.pow(2).sum(-1, keepdim=True) + 1e-6) * (q.shape[-1] ** -0.5)).to(q.dtype)
    k_n = (kf * torch.rsqrt(kf.pow(2).sum(-1, keepdim=True) + 1e-6)).to(k.dtype)
    beta = torch.sigmoid(b.float())
    g = -torch.exp(a_log.float()).unsqueeze(0) * F.softplus(a.float() + dt_bias.float().unsqueeze(0))
    return q_n, k_n, beta, g


def gdn_gated_rmsnorm(x: torch.Tensor, z: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """x * rsqrt(mean(x^2) + 1e-6) * weight * silu(z) per head (triton_kernels/gdn_gated_rmsnorm.py:54-67)."""
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6) * weight.float() * F.silu(z.float())).to(x.dtype)
