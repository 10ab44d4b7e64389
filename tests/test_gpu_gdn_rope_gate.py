"""GPU parity of the Gated-DeltaNet recurrence (decode + token-serial prefill), partial RoPE and gate-pack.

Bars: bf16 outputs within max-abs 2e-2 of the fp32 oracle (in practice one bf16 ulp); fp32 GDN state within
1e-3 relative after 512 decode steps; RoPE pass-through dims byte-equal.
"""
import pytest
import torch

from helpers import bf16_randn, gdn_inputs, maxabs
from oracle import reference_ops as O

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def ops():
    from b200attn import ops as _ops
    return _ops


# --------------------------------------------------------------------------- rope / gate
def test_partial_rope_golden(ops, golden):
    g = golden("partial_rope")
    out = ops.partial_rope(g["a.x"].to(DEV), g["a.ids"].to(DEV), g["a.inv_freq"].to(DEV), 64)
    assert maxabs(out, g["a.out"]) <= 2 ** -6
    assert torch.equal(out.cpu()[..., 64:], g["a.out"][..., 64:])
    xb = g["b.x_thd"].to(DEV).unsqueeze(0).permute(0, 2, 1, 3)
    out = ops.partial_rope(xb, g["b.ids"].to(DEV), g["a.inv_freq"].to(DEV), 64)
    assert out.shape == g["b.out"].shape and maxabs(out, g["b.out"]) <= 2 ** -6
    assert (out.cpu() != g["b.out"]).float().mean().item() < 0.01
    out = ops.partial_rope(g["c.x"].to(DEV), g["c.ids"].to(DEV), g["c.inv_freq"].to(DEV), 96)
    assert maxabs(out, g["c.out"]) <= 2 ** -6
    assert torch.equal(out.cpu()[..., 96:], g["c.out"][..., 96:])


def test_partial_rope_large_positions(ops):
    gen = torch.Generator().manual_seed(12)
    x = bf16_randn(4, 8, 3, 256, gen=gen)
    ids = torch.tensor([[0, 1, 2], [4093, 4094, 4095], [32766, 32767, 32768], [100000, 7, 65535]], dtype=torch.int64)
    inv = (1.0 / (1e7 ** (torch.arange(0, 64, 2, dtype=torch.float32) / 64))).contiguous()
    out = ops.partial_rope(x.to(DEV), ids.to(DEV), inv.to(DEV), 64)
    ref = O.partial_rope(x, ids, inv, 64)
    assert maxabs(out, ref) <= 2 ** -5  # one bf16 ulp at |x| < 8
    assert (out.cpu() != ref).float().mean().item() < 0.01


def test_gate_pack_golden(ops, golden):
    g = golden("gate_pack")
    t, h, d = g["ctx_thd"].shape
    x4 = g["ctx_thd"].to(DEV).permute(1, 0, 2).unsqueeze(0)
    g4 = g["gate"].to(DEV).view(1, t, h, d).permute(0, 2, 1, 3)
    out = ops.attention_gate_pack(x4, g4)
    assert out.shape == g["out"].shape and out.is_contiguous()
    assert maxabs(out, g["out"]) <= 2 ** -7


def test_gate_pack_rejects_batch(ops):
    x = torch.zeros(2, 8, 3, 256, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(AssertionError):
        ops.attention_gate_pack(x, x)


# --------------------------------------------------------------------------- GDN
def test_gdn_decode_golden(ops, golden):
    g = golden("gdn_decode")
    state = g["state_in"].to(DEV)
    # v as a strided view with row stride 3*H*DV, like the slice of the conv output the runner passes
    b, h, dv = g["v"].shape
    storage = torch.zeros(b, 3 * h * dv, dtype=torch.bfloat16, device=DEV)
    storage[:, 2 * h * dv:] = g["v"].to(DEV).reshape(b, h * dv)
    v = storage[:, 2 * h * dv:].view(b, h, dv)
    out = ops.gdn_recurrent_decode(g["q"].to(DEV), g["k"].to(DEV), v, g["beta"].to(DEV), g["g"].to(DEV), state)
    assert maxabs(out, g["out"]) <= 2 ** -8
    assert maxabs(state, g["state_out"]) < 1e-5


def test_gdn_sequential_golden(ops, golden):
    g = golden("gdn_sequential")
    args = [g[k].to(DEV) for k in ("q", "k", "v", "beta", "g")]
    out, state = ops.gdn_recurrent_prefill_sequential(*args, g["cu_seqlens"].to(DEV))
    assert maxabs(out, g["out"]) <= 2 ** -8
    assert maxabs(state, g["state"]) < 1e-5
    out1, state1 = ops.gdn_recurrent_prefill_sequential(*[a[:4] for a in args])
    assert state1.shape == (2, 128, 128)
    out2, state2 = ops.gdn_recurrent_prefill_sequential(*[a[:4] for a in args],
                                                        torch.tensor([0, 4], dtype=torch.int32, device=DEV))
    assert torch.equal(out1, out2) and torch.equal(state1, state2[0])  # None == [0, T], byte for byte


@pytest.mark.parametrize("lengths", [[1], [3], [17], [65], [5, 40, 1, 130]])
def test_gdn_sequential_vs_oracle(ops, lengths):
    gen = torch.Generator().manual_seed(50 + sum(lengths))
    total, heads = sum(lengths), 16
    q, k, v, beta, g = gdn_inputs(total, heads, gen, v_row_stride=3 * heads * 128)
    cu = torch.tensor([0] + list(torch.tensor(lengths).cumsum(0)), dtype=torch.int32)
    ref_out, ref_state = O.gdn_recurrent_prefill_sequential(q, k, v, beta, g, cu)
    storage = torch.zeros(total, 3 * heads * 128, dtype=torch.bfloat16, device=DEV)
    storage[:, 2 * heads * 128:] = v.to(DEV).reshape(total, -1)
    vd = storage[:, 2 * heads * 128:].view(total, heads, 128)
    out, state = ops.gdn_recurrent_prefill_sequential(q.to(DEV), k.to(DEV), vd, beta.to(DEV), g.to(DEV), cu.to(DEV))
    assert maxabs(out, ref_out) <= 1e-2
    assert maxabs(state, ref_state) <= 2e-4


def test_gdn_prefill_then_decode_equals_full_prefill(ops):
    """prefill 17 tokens + 48 decode steps == prefill of all 65 (gdn_recurrent_prefill.py:1628-1674)."""
    gen = torch.Generator().manual_seed(61)
    heads, total, split = 16, 65, 17
    q, k, v, beta, g = (t.to(DEV) for t in gdn_inputs(total, heads, gen))
    full_out, full_state = ops.gdn_recurrent_prefill_sequential(q, k, v, beta, g)
    out_a, state = ops.gdn_recurrent_prefill_sequential(q[:split], k[:split], v[:split], beta[:split], g[:split])
    state = state.unsqueeze(0).contiguous()
    outs = [out_a]
    for t in range(split, total):
        outs.append(ops.gdn_recurrent_decode(q[t:t + 1], k[t:t + 1], v[t:t + 1], beta[t:t + 1], g[t:t + 1], state))
    assert maxabs(torch.cat(outs), full_out) <= 2 ** -8
    assert maxabs(state[0], full_state) < 1e-5


def test_gdn_decode_512_steps_state_drift(ops):
    """fp32 state within 1e-3 relative of the oracle after 512 single-token steps."""
    gen = torch.Generator().manual_seed(62)
    batch, heads, steps = 2, 4, 512
    state = torch.zeros(batch, heads, 128, 128, device=DEV)
    ref_state = torch.zeros(batch, heads, 128, 128)
    worst = 0.0
    for _ in range(steps):
        q, k, v, beta, g = gdn_inputs(batch, heads, gen)
        out = ops.gdn_recurrent_decode(q.to(DEV), k.to(DEV), v.to(DEV), beta.to(DEV), g.to(DEV), state)
        ref = O.gdn_recurrent_decode(q, k, v, beta, g, ref_state)
        worst = max(worst, maxabs(out, ref))
    rel = (state.cpu() - ref_state).norm() / ref_state.norm()
    assert rel.item() < 1e-3
    assert maxabs(state, ref_state) < 1e-3 * ref_state.abs().max().item()
    assert worst <= 2e-2
