"""GPU parity at the EXACT shapes and seeds of the benchmark configurations, against the CPU oracle:

  config 2  one full-attention layer decode step, B=256, contexts ~U[512,4096] (seed 1): fused kernel, both page cuts
  config 3  packed varlen causal prefill, B=32, lengths ~U[16,512] (seed 2): drop-in operator and fused layer step
  config 4  Gated-DeltaNet layer: chunk-64 prefill of 32 x 128 packed tokens, then 512 decode steps at B=32
  and the Gated-DeltaNet decode step at 64 x 16 and 256 x 16 (sequence, head) items, which selects the persistent
  TMA-staged kernel.

Bars: page / index work bit-exact, bf16 outputs within max-abs 2e-2 of the fp32 oracle, fp32 state 1e-5 per step and
1e-3 relative after 512 steps.  Cache contents are generated on the GPU (seeded) and copied to the host for the oracle.
"""
import pytest
import torch

from helpers import cdiv, gdn_inputs, maxabs, rope_inv_freq
from oracle import reference_ops as O

pytestmark = pytest.mark.gpu
DEV = "cuda"
TOL = 2e-2
HQ, HKV, D, PAGE = 8, 2, 256, 16


@pytest.fixture(scope="module")
def ops():
    from b200attn import ops as _ops
    return _ops


def no_timeouts():
    import b200attn
    assert b200attn.load().b200_wait_timed_out() == 0, "a kernel gave up waiting for a staged copy"


def packed_table(pages_per_seq, gen, extra=8):
    """Random page table with exactly the pages each sequence needs (rows padded with page 0)."""
    num_pages = sum(pages_per_seq) + extra
    perm = torch.randperm(num_pages, generator=gen)
    table = torch.zeros(len(pages_per_seq), max(pages_per_seq), dtype=torch.int32)
    off = 0
    for i, n in enumerate(pages_per_seq):
        table[i, :n] = perm[off:off + n].to(torch.int32)
        off += n
    return table, num_pages


@pytest.mark.parametrize("partition", [0, 1])
def test_config2_decode_layer_b256_seed1(ops, partition):
    gen = torch.Generator().manual_seed(1)
    lengths = torch.randint(512, 4097, (256,), generator=gen).tolist()       # the benchmark's draw
    batch = len(lengths)
    table, num_pages = packed_table([cdiv(n + 1, PAGE) for n in lengths], gen)
    ggen = torch.Generator(device=DEV).manual_seed(1)
    k_cache = torch.randn(num_pages, HKV, PAGE, D, device=DEV, generator=ggen).to(torch.bfloat16)
    v_cache = torch.randn(num_pages, HKV, PAGE, D, device=DEV, generator=ggen).to(torch.bfloat16)
    q = torch.randn(batch, HQ, D, generator=gen).to(torch.bfloat16)
    k_new = torch.randn(batch, HKV, D, generator=gen).to(torch.bfloat16)
    v_new = torch.randn(batch, HKV, D, generator=gen).to(torch.bfloat16)
    gate = torch.randn(batch, HQ * D, generator=gen).to(torch.bfloat16)
    pos = torch.tensor(lengths, dtype=torch.int64)
    inv = rope_inv_freq()
    kc, vc = k_cache.clone(), v_cache.clone()
    out = ops.fused_decode_attention(q.to(DEV), k_new.to(DEV), v_new.to(DEV), gate.to(DEV), kc, vc, table.to(DEV),
                                     pos.to(DEV), inv.to(DEV), 64, ops.fused_decode_workspace(DEV), partition=partition)
    torch.cuda.synchronize()
    no_timeouts()
    kr, vr = k_cache.cpu(), v_cache.cpu()
    ref = O.fused_decode_attention(q, k_new, v_new, gate, kr, vr, table, pos, inv, 64, exact=True)
    assert maxabs(out, ref) < TOL
    assert torch.equal(vc, vr.to(DEV)), "V pages: appended rows are copies, everything else untouched"
    kr = kr.to(DEV)
    assert (kc.float() - kr.float()).abs().max().item() <= 2 ** -6      # rotated rows: one bf16 ulp at |x| < 4
    assert (kc != kr).float().mean().item() < 1e-5


def test_config3_packed_prefill_b32_seed2(ops):
    gen = torch.Generator().manual_seed(2)
    lengths = torch.randint(16, 513, (32,), generator=gen).tolist()           # the benchmark's draw: 8275 tokens
    total = sum(lengths)
    q = torch.randn(total, HQ, D, generator=gen).to(torch.bfloat16)
    k = torch.randn(total, HKV, D, generator=gen).to(torch.bfloat16)
    v = torch.randn(total, HKV, D, generator=gen).to(torch.bfloat16)
    gate = torch.randn(total, HQ * D, generator=gen).to(torch.bfloat16)
    table, num_pages = packed_table([cdiv(n, PAGE) for n in lengths], gen)
    k_cache = torch.randn(num_pages, HKV, PAGE, D, generator=gen).to(torch.bfloat16)
    v_cache = torch.randn(num_pages, HKV, PAGE, D, generator=gen).to(torch.bfloat16)
    cu, max_len = ops.build_cu_seqlens(lengths, device="cpu")
    ids = torch.cat([torch.arange(n) for n in lengths]).to(torch.int32)
    inv = rope_inv_freq()
    # drop-in operator on already rotated inputs
    out = ops.gqa_attention_varlen_causal(q.to(DEV), k.to(DEV), v.to(DEV), cu.to(DEV), max_len)
    assert maxabs(out, O.varlen_causal_exact(q, k, v, cu)) < TOL
    # fused layer step: rope + attention + gate + scatter
    kc, vc = k_cache.to(DEV), v_cache.to(DEV)
    fused = ops.fused_prefill_attention(q.to(DEV), k.to(DEV), v.to(DEV), gate.to(DEV), kc, vc, table.to(DEV), cu.to(DEV),
                                        ids.to(DEV), inv.to(DEV), 64, max_len)
    torch.cuda.synchronize()
    no_timeouts()
    kr, vr = k_cache.clone(), v_cache.clone()
    ref = O.fused_prefill_attention(q, k, v, gate, kr, vr, table, cu, ids.view(1, -1), inv, 64, exact=True)
    assert maxabs(fused, ref) < TOL
    assert torch.equal(vc.cpu(), vr), "V pages: scattered rows are copies, slots past a sequence end keep their bytes"
    assert maxabs(kc, kr) <= 2 ** -6
    assert (kc.cpu() != kr).float().mean().item() < 1e-3


def _flat_step(state, q, k, v, beta, g):
    """One oracle delta-rule step for every (sequence, head) at once: the oracle's per-head step over B*H 'heads'."""
    b, h = q.shape[:2]
    new_state, o = O.gdn_step(state.flatten(0, 1), q.flatten(0, 1), k.flatten(0, 1), v.flatten(0, 1), beta.flatten(),
                              g.flatten())
    return new_state.view(b, h, 128, 128), o.view(b, h, 128)


@pytest.mark.parametrize("batch", [64, 256])
def test_gdn_decode_persistent_kernel_vs_oracle(ops, batch):
    """64 x 16 and 256 x 16 items: at least six per SM, which selects the persistent TMA-staged form of the operator.
    v arrives as the runner passes it: a [B,16,128] view with row stride 6144 (a column slice of the conv output)."""
    heads = 16
    gen = torch.Generator().manual_seed(700 + batch)
    q, k, v, beta, g = gdn_inputs(batch, heads, gen, v_row_stride=3 * heads * 128)
    assert v.stride(0) == 6144
    state = torch.randn(batch, heads, 128, 128, generator=gen) * 0.1
    sd = state.to(DEV)
    vd = torch.zeros(batch, 6144, dtype=torch.bfloat16, device=DEV)
    vd[:, 6144 - heads * 128:] = v.reshape(batch, heads * 128).to(DEV)
    v_view = vd[:, 6144 - heads * 128:].view(batch, heads, 128)
    out = ops.gdn_recurrent_decode(q.to(DEV), k.to(DEV), v_view, beta.to(DEV), g.to(DEV), sd)
    torch.cuda.synchronize()
    no_timeouts()
    ref_state, ref_out = _flat_step(state, q, k, v, beta, g)
    assert maxabs(out, ref_out) <= TOL
    assert maxabs(sd, ref_state) <= 1e-5
    # a second step on the updated state (the ring buffers are reused)
    q2, k2, v2, beta2, g2 = gdn_inputs(batch, heads, gen)
    out2 = ops.gdn_recurrent_decode(q2.to(DEV), k2.to(DEV), v2.to(DEV), beta2.to(DEV), g2.to(DEV), sd)
    ref_state2, ref_out2 = _flat_step(ref_state, q2, k2, v2, beta2, g2)
    assert maxabs(out2, ref_out2) <= TOL
    assert maxabs(sd, ref_state2) <= 2e-5


@pytest.mark.parametrize("form", [0, 1, 2, 3])
@pytest.mark.parametrize("batch", [3, 40])
def test_gdn_decode_every_kernel_form(ops, form, batch):
    """The operator has three kernel forms (one CTA per head, one warp per 32 columns, a persistent ring of tensor-map
    TMA boxes) and picks by size (form 0); here each is pinned in turn and checked against the oracle, two steps in a
    row, with the strided `v` view of the runner."""
    from b200attn import _lib
    heads = 16
    gen = torch.Generator().manual_seed(900 + batch)
    q, k, v, beta, g = gdn_inputs(batch, heads, gen, v_row_stride=3 * heads * 128)
    state = torch.randn(batch, heads, 128, 128, generator=gen) * 0.1
    sd = state.to(DEV)
    vd = torch.zeros(batch, 6144, dtype=torch.bfloat16, device=DEV)
    vd[:, 6144 - heads * 128:] = v.reshape(batch, heads * 128).to(DEV)
    v_view = vd[:, 6144 - heads * 128:].view(batch, heads, 128)
    _lib.call("b200_gdn_recurrent_decode_form", form)
    try:
        out = ops.gdn_recurrent_decode(q.to(DEV), k.to(DEV), v_view, beta.to(DEV), g.to(DEV), sd)
        ref_state, ref_out = _flat_step(state, q, k, v, beta, g)
        assert maxabs(out, ref_out) <= TOL and maxabs(sd, ref_state) <= 1e-5
        q2, k2, v2, beta2, g2 = gdn_inputs(batch, heads, gen)
        out2 = ops.gdn_recurrent_decode(q2.to(DEV), k2.to(DEV), v2.to(DEV), beta2.to(DEV), g2.to(DEV), sd)
        ref_state2, ref_out2 = _flat_step(ref_state, q2, k2, v2, beta2, g2)
        assert maxabs(out2, ref_out2) <= TOL and maxabs(sd, ref_state2) <= 2e-5
    finally:
        _lib.call("b200_gdn_recurrent_decode_form", 0)
    torch.cuda.synchronize()
    no_timeouts()


@pytest.mark.parametrize("form", [0, 2, 3])
def test_gdn_decode_state_inside_a_larger_buffer(ops, form):
    """A recurrent state that is a view into a wider allocation (one spare head per sequence) is not the dense layout
    the ring form needs: the size-based choice takes the one-warp slices, a pinned ring falls back to one CTA per head.
    The spare heads must stay untouched."""
    from b200attn import _lib
    batch, heads = 5, 16
    gen = torch.Generator().manual_seed(321)
    q, k, v, beta, g = gdn_inputs(batch, heads, gen)
    state = torch.randn(batch, heads, 128, 128, generator=gen) * 0.1
    wide = torch.full((batch, heads + 1, 128, 128), 7.0, device=DEV)
    wide[:, :heads] = state.to(DEV)
    view = wide[:, :heads]
    assert not view.is_contiguous()
    _lib.call("b200_gdn_recurrent_decode_form", form)
    try:
        out = ops.gdn_recurrent_decode(q.to(DEV), k.to(DEV), v.to(DEV), beta.to(DEV), g.to(DEV), view)
    finally:
        _lib.call("b200_gdn_recurrent_decode_form", 0)
    ref_state, ref_out = _flat_step(state, q, k, v, beta, g)
    assert maxabs(out, ref_out) <= TOL and maxabs(view, ref_state) <= 1e-5
    assert bool((wide[:, heads] == 7.0).all())
    torch.cuda.synchronize()
    no_timeouts()


def test_config4_gdn_layer_prefill_then_512_decode_steps(ops):
    """Chunk-64 prefill over 32 packed prompts of 128 tokens on the tensor cores against the oracle's chunk pipeline,
    then 512 single-token steps at B=32 from that state against the oracle recurrence (fresh inputs per step, seed 3):
    out within 2e-2 at every step, state within 1e-3 relative at the end."""
    heads, batch, prompt = 16, 32, 128
    gen = torch.Generator().manual_seed(3)
    total = batch * prompt
    q, k, v, beta, g = gdn_inputs(total, heads, gen, v_row_stride=3 * heads * 128)
    cu = torch.arange(batch + 1, dtype=torch.int32) * prompt
    vd = torch.zeros(total, 6144, dtype=torch.bfloat16, device=DEV)
    vd[:, 6144 - heads * 128:] = v.reshape(total, heads * 128).to(DEV)
    out, state = ops.gdn_chunked_prefill_packed(q.to(DEV), k.to(DEV), vd[:, 6144 - heads * 128:].view(total, heads, 128),
                                                beta.to(DEV), g.to(DEV), cu.to(DEV))
    torch.cuda.synchronize()
    no_timeouts()
    ref_out, ref_state = O.gdn_chunked_prefill_packed(q, k, v, beta, g, cu)
    assert maxabs(out, ref_out) <= 1e-2          # the reference's own chunked-vs-sequential bar
    assert maxabs(state, ref_state) <= 5e-4
    seq_out, seq_state = ops.gdn_recurrent_prefill_sequential(q.to(DEV), k.to(DEV), v.to(DEV), beta.to(DEV), g.to(DEV),
                                                              cu.to(DEV))
    assert maxabs(out, seq_out) <= 1e-2 and maxabs(state, seq_state) <= 5e-4
    worst = 0.0
    for step in range(512):
        qs, ks, vs, bs, gs = gdn_inputs(batch, heads, gen)
        o = ops.gdn_recurrent_decode(qs.to(DEV), ks.to(DEV), vs.to(DEV), bs.to(DEV), gs.to(DEV), state)
        ref_state, ro = _flat_step(ref_state, qs, ks, vs, bs, gs)
        if step % 16 == 0 or step == 511:
            worst = max(worst, maxabs(o, ro))
    assert worst <= TOL, worst
    rel = (state.cpu() - ref_state).norm().item() / ref_state.norm().item()
    assert rel <= 1e-3, rel
    assert maxabs(state, ref_state) <= 1e-3 * ref_state.abs().max().item() + 1e-5
    no_timeouts()


def test_bounded_wait_gives_up_without_harm():
    """A staged-copy wait that nothing will ever complete runs out, sets the library's flag, leaves the output alone
    and the context usable: the path every kernel takes when a copy does not arrive."""
    import b200attn
    from b200attn import _lib
    lib = b200attn.load()
    torch.cuda.synchronize()
    assert lib.b200_wait_timed_out() == 0
    sentinel = torch.full((1,), 12345, dtype=torch.int32, device=DEV)
    _lib.call("b200_selftest_wait_timeout", sentinel.data_ptr(), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert int(sentinel) == 12345
    assert lib.b200_wait_timed_out() == 1
    assert lib.b200_wait_timed_out() == 0          # reading the flag clears it
    x = torch.arange(8, device=DEV)                # the context still works
    assert int(x.sum()) == 28
