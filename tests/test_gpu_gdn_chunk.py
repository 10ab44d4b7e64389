"""GPU parity of the chunk-64 Gated-DeltaNet operators (prepare_wy / chunk_state / chunk_output).

Bars are the reference's own (gdn_recurrent_prefill.py:1520-1526, :1456-1470): w, u 2e-4; g_cumsum 1e-6 relative;
chunked vs token-serial: out 1e-2, state 5e-4.
"""
import pytest
import torch

from helpers import gdn_inputs, maxabs
from oracle import reference_ops as O

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def ops():
    from b200attn import ops as _ops
    return _ops


def test_chunk_ops_golden(ops, golden):
    g = golden("gdn_chunked")
    d = {k: v.to(DEV) for k, v in g.items()}
    w, u, gcs = ops.gdn_chunk_prepare_wy(d["k"], d["v"], d["beta"], d["g"])
    assert maxabs(gcs, g["g_cumsum"]) < 2e-6 * g["g_cumsum"].abs().max().item()
    assert maxabs(w, g["w"]) < 2e-4 and maxabs(u, g["u_base"]) < 2e-4
    delta, cs, fs = ops.gdn_chunk_state(d["k"], d["w"], d["u_base"], d["g_cumsum"])
    assert maxabs(delta, g["delta"]) < 2e-4
    assert maxabs(cs, g["chunk_state"]) < 2e-4 and maxabs(fs, g["final_state"]) < 2e-4
    out = ops.gdn_chunk_output(d["q"], d["k"], d["delta"], d["g_cumsum"], d["chunk_state"])
    assert out.shape == g["out"].shape and maxabs(out, g["out"]) <= 1e-2
    out2, fs2 = ops.call_gdn_recurrent_prefill_chunked_triton(d["q"], d["k"], d["v"], d["beta"], d["g"])
    assert maxabs(out2, g["seq_out"]) < 1e-2 and maxabs(fs2, g["seq_state"]) < 5e-4


@pytest.mark.parametrize("token_num", [1, 3, 63, 64, 65, 129, 512, 1025])
def test_chunked_vs_sequential(ops, token_num):
    """The reference's length grid (gdn_recurrent_prefill.py:1390): chunk pipeline == token-serial kernel, with
    strided q/k/v views as the runner passes them."""
    gen = torch.Generator().manual_seed(900 + token_num)
    heads = 16
    q, k, v, beta, g = gdn_inputs(token_num, heads, gen)
    storage = torch.zeros(token_num, 3 * heads * 128, dtype=torch.bfloat16, device=DEV)
    storage[:, : heads * 128] = q.to(DEV).reshape(token_num, -1)
    storage[:, heads * 128: 2 * heads * 128] = k.to(DEV).reshape(token_num, -1)
    storage[:, 2 * heads * 128:] = v.to(DEV).reshape(token_num, -1)
    qd = storage[:, : heads * 128].view(token_num, heads, 128)
    kd = storage[:, heads * 128: 2 * heads * 128].view(token_num, heads, 128)
    vd = storage[:, 2 * heads * 128:].view(token_num, heads, 128)
    out_c, state_c = ops.call_gdn_recurrent_prefill_chunked_triton(qd, kd, vd, beta.to(DEV), g.to(DEV))
    out_s, state_s = ops.gdn_recurrent_prefill_sequential(qd, kd, vd, beta.to(DEV), g.to(DEV))
    assert torch.isfinite(out_c.float()).all() and torch.isfinite(state_c).all()
    assert maxabs(out_c, out_s) <= 1e-2
    assert maxabs(state_c, state_s) <= 5e-4
    if token_num <= 129:
        ref_out, ref_state = O.gdn_recurrent_prefill_sequential(q, k, v, beta, g)
        assert maxabs(out_c, ref_out) <= 1e-2 and maxabs(state_c, ref_state) <= 5e-4


def test_prepare_wy_vs_oracle(ops):
    gen = torch.Generator().manual_seed(77)
    q, k, v, beta, g = gdn_inputs(200, 4, gen)
    w, u, gcs = ops.gdn_chunk_prepare_wy(k.to(DEV), v.to(DEV), beta.to(DEV), g.to(DEV))
    rw, ru, rg = O.gdn_chunk_prepare_wy(k, v, beta, g)
    assert maxabs(gcs, rg) < 2e-6 * rg.abs().max().item()
    assert maxabs(w, rw) < 2e-4 and maxabs(u, ru) < 2e-4


@pytest.mark.parametrize("fused", [True, False], ids=["tcgen05", "three-stage"])
@pytest.mark.parametrize("lengths", [[128] * 4, [5, 64, 65, 1, 200], [130], [63, 300, 17]])
def test_chunked_prefill_packed(ops, lengths, fused):
    """Packed chunk-64 prefill (32 prompts in one call, which the reference cannot run in one call), as the single
    tcgen05 kernel and as the three reference-shaped stages: pinned by (i) the token-serial kernel with cu_seqlens
    and (ii) the oracle's per-sequence chunk pipeline."""
    gen = torch.Generator().manual_seed(1200 + sum(lengths))
    heads, total = 16, sum(lengths)
    q, k, v, beta, g = gdn_inputs(total, heads, gen, v_row_stride=3 * heads * 128)
    cu = torch.tensor([0] + list(torch.tensor(lengths).cumsum(0)), dtype=torch.int32)
    storage = torch.zeros(total, 3 * heads * 128, dtype=torch.bfloat16, device=DEV)
    storage[:, 2 * heads * 128:] = v.to(DEV).reshape(total, -1)
    vd = storage[:, 2 * heads * 128:].view(total, heads, 128)
    qd, kd, bd, gd, cud = q.to(DEV), k.to(DEV), beta.to(DEV), g.to(DEV), cu.to(DEV)
    out_c, state_c = ops.gdn_chunked_prefill_packed(qd, kd, vd, bd, gd, cud, max(lengths), fused=fused)
    out_s, state_s = ops.gdn_recurrent_prefill_sequential(qd, kd, vd, bd, gd, cud)
    assert out_c.shape == out_s.shape and state_c.shape == state_s.shape == (len(lengths), heads, 128, 128)
    assert torch.isfinite(out_c.float()).all() and torch.isfinite(state_c).all()
    assert maxabs(out_c, out_s) <= 1e-2 and maxabs(state_c, state_s) <= 5e-4
    if total <= 400:
        ref_out, ref_state = O.gdn_chunked_prefill_packed(q, k, v, beta, g, cu)
        assert maxabs(out_c, ref_out) <= 1e-2 and maxabs(state_c, ref_state) <= 5e-4


@pytest.mark.parametrize("lengths", [[128] * 32, [1000, 513, 64, 2048]])
def test_fused_chunk_prefill_long(ops, lengths):
    """The tcgen05 chunk kernel at the batched-prompt size (32 x 128) and over many chunks per sequence (the state is
    carried in tensor memory for up to 32 chunks) against the token-serial kernel; no bounded wait may run out."""
    from b200attn import _lib
    gen = torch.Generator().manual_seed(4242 + len(lengths))
    heads, total = 16, sum(lengths)
    q, k, v, beta, g = gdn_inputs(total, heads, gen)
    cu = torch.tensor([0] + list(torch.tensor(lengths).cumsum(0)), dtype=torch.int32)
    qd, kd, vd, bd, gd, cud = (x.to(DEV) for x in (q, k, v, beta, g, cu))
    out_c, state_c = ops.gdn_chunked_prefill_packed(qd, kd, vd, bd, gd, cud)
    out_s, state_s = ops.gdn_recurrent_prefill_sequential(qd, kd, vd, bd, gd, cud)
    torch.cuda.synchronize()
    assert _lib.load().b200_wait_timed_out() == 0
    assert torch.isfinite(out_c.float()).all() and torch.isfinite(state_c).all()
    assert maxabs(out_c, out_s) <= 1e-2 and maxabs(state_c, state_s) <= 5e-4


@pytest.mark.parametrize("token_num", [65, 200, 1100])
def test_chunk_stages_on_unaligned_views(ops, token_num):
    """q/k/v as column views of a buffer whose row stride is not a multiple of 8 elements and whose columns start two
    elements in: the three stages then stage their rows element by element (no 16-byte loads), the single-sequence
    entry point routes such inputs to them at every length, and the results still match the token-serial kernel."""
    gen = torch.Generator().manual_seed(7000 + token_num)
    heads = 16
    q, k, v, beta, g = gdn_inputs(token_num, heads, gen)
    width = 3 * heads * 128
    storage = torch.zeros(token_num, width + 6, dtype=torch.bfloat16, device=DEV)
    storage[:, 2: 2 + width] = torch.cat([q.reshape(token_num, -1), k.reshape(token_num, -1),
                                          v.reshape(token_num, -1)], dim=1).to(DEV)
    qd = storage[:, 2: 2 + heads * 128].view(token_num, heads, 128)
    kd = storage[:, 2 + heads * 128: 2 + 2 * heads * 128].view(token_num, heads, 128)
    vd = storage[:, 2 + 2 * heads * 128: 2 + width].view(token_num, heads, 128)
    assert qd.stride(0) % 8 != 0 and qd.data_ptr() % 16 != 0
    out_c, state_c = ops.call_gdn_recurrent_prefill_chunked_triton(qd, kd, vd, beta.to(DEV), g.to(DEV))
    out_s, state_s = ops.gdn_recurrent_prefill_sequential(qd, kd, vd, beta.to(DEV), g.to(DEV))
    assert torch.isfinite(out_c.float()).all() and torch.isfinite(state_c).all()
    assert maxabs(out_c, out_s) <= 1e-2 and maxabs(state_c, state_s) <= 5e-4
    w, u, gcs = ops.gdn_chunk_prepare_wy(kd, vd, beta.to(DEV), g.to(DEV))
    w2, u2, gcs2 = ops.gdn_chunk_prepare_wy(k.to(DEV), v.to(DEV), beta.to(DEV), g.to(DEV))
    assert torch.equal(w, w2) and torch.equal(u, u2) and torch.equal(gcs, gcs2)
