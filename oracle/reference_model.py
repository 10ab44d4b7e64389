"""TEST INFRASTRUCTURE ONLY - an fp32 CPU restatement of the reference runner's forward pass
(engine/runner.py:212-405 prefill mixers, :408-571 decode step, which compute the same function of the token
history) for the Qwen3.5-0.8B architecture.  It recomputes the whole history for every query (no caches, no pages, no
chunking), so it is independent of every caching / paging / position decision the CUDA engine makes.  Everything is
fp32; the weights are the engine's bf16 weights widened exactly.  Only tests may import this module.

Parity status: the per-operator oracle (reference_ops.py) is pinned against the reference's own kernels; this
model-level restatement is pinned only through those operators' math (the reference's whole model cannot run in the
Triton interpreter: its residual_add adds raw bf16 bit patterns there, and no checkpoint exists offline).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .reference_ops import gdn_step


def widen(weights: dict, device="cpu") -> dict:
    """The engine's weight dictionary in fp32, on the CPU by default (`device` lets a GPU test run the same eager fp32
    arithmetic on the device when the model is too large for the host to finish in seconds)."""
    def conv(v):
        if isinstance(v, torch.Tensor):
            return v.detach().float().to(device)
        if isinstance(v, list):
            return [conv(x) for x in v]
        if isinstance(v, dict):
            return {k: conv(x) for k, x in v.items()}
        return v
    return conv(weights)


def _rms(x, weight, eps):
    """triton_kernels/qwen_rmsnorm.py:70-73."""
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * (1.0 + weight)


def _gdn_layer(cfg, layer, h):
    """engine/runner.py:212-330 (`_gdn`), one sequence, zero initial conv and recurrent state."""
    total, heads, dim, kd = h.shape[0], cfg.gdn_heads, cfg.gdn_dim, cfg.gdn_width
    fused = h @ layer["in_proj"].t()
    qkv, z = fused[:, : 3 * kd], fused[:, 3 * kd: 4 * kd]
    a, b = fused[:, 4 * kd: 4 * kd + heads], fused[:, 4 * kd + heads:]
    padded = F.pad(qkv, (0, 0, 3, 0))
    conv = sum(padded[r: r + total] * layer["conv"][:, r] for r in range(4))  # depthwise_causal_conv4_prefill.py:18-91
    conv = F.silu(conv)
    q = conv[:, :kd].view(total, heads, dim)
    k = conv[:, kd: 2 * kd].view(total, heads, dim)
    v = conv[:, 2 * kd:].view(total, heads, dim)
    q = q * torch.rsqrt(q.pow(2).sum(-1, keepdim=True) + 1e-6) * dim ** -0.5     # gdn_qk_norm_gates.py:68-69
    k = k * torch.rsqrt(k.pow(2).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(b)
    g = -torch.exp(layer["a_log"]).unsqueeze(0) * F.softplus(a + layer["dt_bias"].unsqueeze(0))
    state = torch.zeros(heads, dim, dim, device=h.device)
    core = torch.empty(total, heads, dim, device=h.device)
    for t in range(total):
        state, core[t] = gdn_step(state, q[t], k[t], v[t], beta[t], g[t])
    normed = core * torch.rsqrt(core.pow(2).mean(-1, keepdim=True) + 1e-6) * layer["norm"] * \
        F.silu(z.reshape(total, heads, dim))                                         # gdn_gated_rmsnorm.py:54-67
    return normed.reshape(total, kd) @ layer["out_proj"].t()


def _attention_layer(cfg, layer, h):
    """engine/runner.py:332-405 (`_attention`), one sequence."""
    total, nq, nkv, d = h.shape[0], cfg.num_q_heads, cfg.num_kv_heads, cfg.head_dim
    qd, kvd = nq * d, nkv * d
    fused = h @ layer["qkvg"].t()
    q = _rms(fused[:, :qd].view(total, nq, d), layer["q_norm"], cfg.eps)
    gate = fused[:, qd: 2 * qd]
    k = _rms(fused[:, 2 * qd: 2 * qd + kvd].view(total, nkv, d), layer["k_norm"], cfg.eps)
    v = fused[:, 2 * qd + kvd:].view(total, nkv, d)
    half = cfg.rotary_dim // 2
    inv_freq = 1.0 / (cfg.rope_theta ** (torch.arange(0, cfg.rotary_dim, 2, dtype=torch.float32, device=h.device) / cfg.rotary_dim))
    ang = torch.arange(total, dtype=torch.float32, device=h.device).unsqueeze(1) * inv_freq.unsqueeze(0)   # partial_rope.py:56-132
    cos, sin = torch.cos(ang).unsqueeze(1), torch.sin(ang).unsqueeze(1)

    def rope(x):
        first, second = x[..., :half], x[..., half: cfg.rotary_dim]
        return torch.cat((first * cos - second * sin, first * sin + second * cos, x[..., cfg.rotary_dim:]), dim=-1)

    q, k = rope(q), rope(k)
    k = k.repeat_interleave(nq // nkv, dim=1)
    v = v.repeat_interleave(nq // nkv, dim=1)
    scores = torch.einsum("thd,shd->hts", q, k) * d ** -0.5
    mask = torch.ones(total, total, dtype=torch.bool, device=h.device).tril()
    probs = torch.softmax(scores.masked_fill(~mask, float("-inf")), dim=-1)
    ctx = torch.einsum("hts,shd->thd", probs, v).reshape(total, qd)
    return (ctx * torch.sigmoid(gate)) @ layer["o_proj"].t()                         # attention_gate_pack.py:46-64


def all_hidden(cfg, w32: dict, tokens: list[int]) -> torch.Tensor:
    """Final-norm hidden state [T, hidden] at EVERY position of one sequence (the model is causal: row t depends on
    tokens[:t+1] only), i.e. what the runner feeds its LM head after consuming token t."""
    x = w32["embed"][torch.tensor(tokens, dtype=torch.long, device=w32["embed"].device)]
    for layer in w32["layers"]:
        h = _rms(x, layer["ln1"], cfg.eps)
        mixed = _gdn_layer(cfg, layer, h) if layer["kind"] == "gdn" else _attention_layer(cfg, layer, h)
        x = x + mixed
        h = _rms(x, layer["ln2"], cfg.eps)
        gate_up = h @ layer["gate_up"].t()
        x = x + (F.silu(gate_up[:, : cfg.intermediate]) * gate_up[:, cfg.intermediate:]) @ layer["down"].t()
    return _rms(x, w32["norm"], cfg.eps)


def last_token_logits(cfg, w32: dict, tokens: list[int]) -> torch.Tensor:
    """Logits [vocab] for the token that follows `tokens` (full recomputation)."""
    x = w32["embed"][torch.tensor(tokens, dtype=torch.long, device=w32["embed"].device)]
    for layer in w32["layers"]:
        h = _rms(x, layer["ln1"], cfg.eps)
        mixed = _gdn_layer(cfg, layer, h) if layer["kind"] == "gdn" else _attention_layer(cfg, layer, h)
        x = x + mixed
        h = _rms(x, layer["ln2"], cfg.eps)
        gate_up = h @ layer["gate_up"].t()
        x = x + (F.silu(gate_up[:, : cfg.intermediate]) * gate_up[:, cfg.intermediate:]) @ layer["down"].t()
    return _rms(x[-1], w32["norm"], cfg.eps) @ w32["embed"].t()
