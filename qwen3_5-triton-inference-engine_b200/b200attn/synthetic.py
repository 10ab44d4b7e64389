"""Seeded synthetic inputs for the attention / Gated-DeltaNet operators (CPU tensors; callers move them to the GPU):
paged decode cases with a shuffled page table and random bytes everywhere, Gated-DeltaNet inputs with the value
distributions the model's own gate / norm operators produce.  Used by the smoke check, the benchmark and the tests."""
from __future__ import annotations

import torch

PAGE = 16


def bf16_randn(*shape, gen):
    return torch.randn(*shape, generator=gen, dtype=torch.float32).to(torch.bfloat16)


def cdiv(a, b):
    return (a + b - 1) // b


def make_paged_case(lengths, *, seed, hq=8, hkv=2, d=256, extra_pages=5, slack_tokens=1):
    """Paged decode inputs for contexts `lengths` (tokens already cached; the step appends one more).
    Page table is a random permutation; cache contents are random everywhere (also in unowned pages and in
    slots past each context) so stale data cannot pass for zeros."""
    gen = torch.Generator().manual_seed(seed)
    batch = len(lengths)
    pps = max(cdiv(n + slack_tokens, PAGE) for n in lengths)
    num_pages = batch * pps + extra_pages
    order = torch.randperm(num_pages, generator=gen)
    block_table = order[: batch * pps].view(batch, pps).to(torch.int32).contiguous()
    return dict(
        block_table=block_table,
        k_cache=bf16_randn(num_pages, hkv, PAGE, d, gen=gen),
        v_cache=bf16_randn(num_pages, hkv, PAGE, d, gen=gen),
        q=bf16_randn(batch, hq, d, gen=gen),
        k_new=bf16_randn(batch, hkv, d, gen=gen),
        v_new=bf16_randn(batch, hkv, d, gen=gen),
        gate=bf16_randn(batch, hq * d, gen=gen),
        pos=torch.tensor(lengths, dtype=torch.int64),
        unowned=order[batch * pps:],
    )


def rope_inv_freq(rotary_dim=64, theta=1e7):
    return (1.0 / (theta ** (torch.arange(0, rotary_dim, 2, dtype=torch.float32) / rotary_dim))).contiguous()


def gdn_inputs(token_num, heads, gen, dk=128, dv=128, v_row_stride=None):
    """q/k L2-normalised per head (q also times dk**-0.5), rounded to bf16; beta = sigmoid(N(0,1));
    g = -softplus(N(0,1)) * exp(A), A ~ U(0, 2.7) per head (the distribution the model's gate kernel produces)."""
    q = torch.randn(token_num, heads, dk, generator=gen)
    k = torch.randn(token_num, heads, dk, generator=gen)
    q = (q * torch.rsqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5).to(torch.bfloat16)
    k = (k * torch.rsqrt((k * k).sum(-1, keepdim=True) + 1e-6)).to(torch.bfloat16)
    if v_row_stride is None:
        v = bf16_randn(token_num, heads, dv, gen=gen)
    else:
        storage = bf16_randn(token_num, v_row_stride, gen=gen)
        v = storage[:, v_row_stride - heads * dv:].view(token_num, heads, dv)
    beta = torch.sigmoid(torch.randn(token_num, heads, generator=gen))
    a = torch.rand(heads, generator=gen) * 2.7
    g = -torch.nn.functional.softplus(torch.randn(token_num, heads, generator=gen)) * torch.exp(a)
    return q, k, v, beta, g


def maxabs(a, b):
    return (a.float().cpu() - b.float().cpu()).abs().max().item()
