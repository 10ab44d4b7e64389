"""GPU parity of the packed varlen causal prefill attention (drop-in operator and fused rope+scatter+gate path).

Bars: bf16 outputs within max-abs 2e-2 of the fp32 oracle (relative to max|ref| like the reference's self-test);
V rows in the cache bit-exact, K rows within one bf16 ulp of the oracle's rotation.
"""
import pytest
import torch

from helpers import bf16_randn, cdiv, maxabs, rope_inv_freq
from oracle import reference_ops as O

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def ops():
    from b200attn import ops as _ops
    return _ops


def rel_to_max(got, ref):
    ref = ref.float().cpu()
    return (got.float().cpu() - ref).abs().max().item() / max(ref.abs().max().item(), 1e-9)


def test_varlen_causal_golden(ops, golden):
    g = golden("varlen_causal")
    out = ops.gqa_attention_varlen_causal(g["q"].to(DEV), g["k"].to(DEV), g["v"].to(DEV), g["cu_seqlens"].to(DEV),
                                          int(g["lengths"].max()))
    assert out.shape == g["out"].shape
    assert maxabs(out, g["out"]) <= 2e-2          # the reference kernel itself (different tile sizes, same rounding points)
    assert (out.float().cpu() - g["out"].float()).abs().mean().item() < 1e-3  # scores are scaled in fp32 here, the reference re-rounds q*scale to bf16
    exact = O.varlen_causal_exact(g["q"], g["k"], g["v"], g["cu_seqlens"])
    assert rel_to_max(out, exact) < 2e-2


@pytest.mark.parametrize("lengths", [[7], [16, 16], [1, 3, 17, 64], [3, 100, 1, 64], [1, 1, 1, 1000], [33, 32, 31, 65, 129],
                                     [512, 16, 300]])
def test_varlen_causal_vs_oracle(ops, lengths):
    """The reference's self-test grid (gqa_attention_varlen_causal.py:359) plus block-boundary lengths."""
    gen = torch.Generator().manual_seed(200 + sum(lengths))
    total = sum(lengths)
    q, k, v = bf16_randn(total, 8, 256, gen=gen), bf16_randn(total, 2, 256, gen=gen), bf16_randn(total, 2, 256, gen=gen)
    cu = torch.tensor([0] + list(torch.tensor(lengths).cumsum(0)), dtype=torch.int32)
    out = ops.gqa_attention_varlen_causal(q.to(DEV), k.to(DEV), v.to(DEV), cu.to(DEV), max(lengths))
    torch.cuda.synchronize()
    import b200attn
    assert b200attn.load().b200_wait_timed_out() == 0
    exact = O.varlen_causal_exact(q, k, v, cu)
    assert torch.isfinite(out.float()).all()
    assert rel_to_max(out, exact) < 2e-2
    assert maxabs(out, exact) < 2e-2 * max(1.0, exact.abs().max().item())


def test_varlen_causal_strided_inputs(ops):
    """q/k/v as slices of fused projection rows (row strides 2048+, not contiguous per token)."""
    gen = torch.Generator().manual_seed(7)
    lengths = [40, 9]
    total = sum(lengths)
    fused = bf16_randn(total, 8 * 256 + 2 * 256 + 2 * 256, gen=gen)
    cu = torch.tensor([0, 40, 49], dtype=torch.int32)
    fd = fused.to(DEV)
    q = fd[:, :2048].view(total, 8, 256)
    k = fd[:, 2048:2560].view(total, 2, 256)
    v = fd[:, 2560:].view(total, 2, 256)
    out = ops.gqa_attention_varlen_causal(q, k, v, cu.to(DEV), 40)
    exact = O.varlen_causal_exact(fused[:, :2048].view(total, 8, 256), fused[:, 2048:2560].view(total, 2, 256),
                                  fused[:, 2560:].view(total, 2, 256), cu)
    assert rel_to_max(out, exact) < 2e-2


@pytest.mark.parametrize("lengths", [[5], [16, 17, 1], [70, 33, 128, 2], [300, 45], [129, 256, 257], [1100]])
def test_fused_prefill_vs_oracle(ops, lengths):
    gen = torch.Generator().manual_seed(400 + sum(lengths))
    total, batch = sum(lengths), len(lengths)
    q, k, v = bf16_randn(total, 8, 256, gen=gen), bf16_randn(total, 2, 256, gen=gen), bf16_randn(total, 2, 256, gen=gen)
    gate = bf16_randn(total, 2048, gen=gen)
    pps = cdiv(max(lengths), 16)
    num_pages = batch * pps + 6
    order = torch.randperm(num_pages, generator=gen)
    bt = order[: batch * pps].view(batch, pps).to(torch.int32).contiguous()
    kc0, vc0 = bf16_randn(num_pages, 2, 16, 256, gen=gen), bf16_randn(num_pages, 2, 16, 256, gen=gen)
    cu = torch.tensor([0] + list(torch.tensor(lengths).cumsum(0)), dtype=torch.int32)
    ids = torch.cat([torch.arange(n) for n in lengths]).to(torch.int32).unsqueeze(0)
    inv = rope_inv_freq()
    kr, vr = kc0.clone(), vc0.clone()
    ref = O.fused_prefill_attention(q, k, v, gate, kr, vr, bt, cu, ids, inv, 64, exact=True)
    kc, vc = kc0.to(DEV), vc0.to(DEV)
    out = ops.fused_prefill_attention(q.to(DEV), k.to(DEV), v.to(DEV), gate.to(DEV), kc, vc, bt.to(DEV), cu.to(DEV),
                                      ids.to(DEV), inv.to(DEV), 64, max(lengths))
    torch.cuda.synchronize()
    assert torch.equal(vc.cpu(), vr)                      # V scatter: bit-exact, untouched slots keep their bytes
    assert maxabs(kc, kr) <= 2 ** -5 and (kc.cpu() != kr).float().mean().item() < 1e-2
    assert torch.equal(kc.cpu()[order[batch * pps:]], kc0[order[batch * pps:]])
    assert maxabs(out, ref) < 2e-2 * max(1.0, ref.float().abs().max().item())


def test_fused_prefill_matches_dropin_chain(ops):
    """fused == partial_rope x2 -> gqa_attention_varlen_causal -> attention_gate_pack -> paged_kv_fill_varlen."""
    gen = torch.Generator().manual_seed(55)
    lengths = [37, 64, 5]
    total, batch = sum(lengths), len(lengths)
    q, k, v = (bf16_randn(total, 8, 256, gen=gen).to(DEV), bf16_randn(total, 2, 256, gen=gen).to(DEV),
               bf16_randn(total, 2, 256, gen=gen).to(DEV))
    gate = bf16_randn(total, 2048, gen=gen).to(DEV)
    pps = cdiv(max(lengths), 16)
    bt = torch.randperm(batch * pps, generator=gen).view(batch, pps).to(torch.int32).to(DEV)
    cu, max_len = ops.build_cu_seqlens(lengths, device=DEV)
    ids = torch.cat([torch.arange(n) for n in lengths]).to(torch.int32).unsqueeze(0).to(DEV)
    inv = rope_inv_freq().to(DEV)
    q4 = ops.partial_rope(q.unsqueeze(0).permute(0, 2, 1, 3), ids, inv, 64)
    k4 = ops.partial_rope(k.unsqueeze(0).permute(0, 2, 1, 3), ids, inv, 64)
    v4 = v.unsqueeze(0).permute(0, 2, 1, 3)
    ctx = ops.gqa_attention_varlen_causal(q4[0].permute(1, 0, 2).contiguous(), k4[0].permute(1, 0, 2).contiguous(),
                                          v4[0].permute(1, 0, 2).contiguous(), cu, max_len).permute(1, 0, 2).unsqueeze(0)
    chain = ops.attention_gate_pack(ctx, gate.view(1, total, 8, 256).permute(0, 2, 1, 3))
    kc1, vc1 = ops.allocate_paged_kv_cache(batch * pps, 2, 256, device=DEV)
    ops.paged_kv_fill_varlen(kc1, vc1, k4[0], v4[0], bt, cu, max_len)
    kc2, vc2 = ops.allocate_paged_kv_cache(batch * pps, 2, 256, device=DEV)
    fused = ops.fused_prefill_attention(q, k, v, gate, kc2, vc2, bt, cu, ids, inv, 64, max_len)
    assert torch.equal(kc1, kc2) and torch.equal(vc1, vc2)
    assert maxabs(fused, chain) <= 2e-2  # two attention kernels (tcgen05 drop-in, fused path), same inputs
