"""GPU parity of the operators AROUND the path against outputs of the REFERENCE's own kernels (tests/golden/glue_*.pt):
the drop-in `wy_lib::*` operators of b200attn/glue_ops.py one by one, and the fused decode-layer kernels
(b200_gdn_decode_prep, b200_gdn_decode_fused, b200_fused_decode_attention_ex with the q/k head norms inside) against
the reference runner's operator chains.  bf16 results: within one bf16 ulp with at most a few per cent of the elements
not bit-equal (transcendentals come from different libraries); byte moves bit-exact; fp32 gates 5e-6 relative."""
import pytest
import torch

from helpers import assert_bf16_close

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def mods():
    from b200attn import glue_ops, ops
    return ops, glue_ops


def dev(g):
    return {k: (v.to(DEV) if isinstance(v, torch.Tensor) else v) for k, v in g.items()}


def test_conv4_operators(mods, golden):
    _, G = mods
    g = dev(golden("glue_conv4"))
    out = G.depthwise_causal_conv4_prefill(g["x"], g["weight"], g["seq_start"])
    assert_bf16_close(out, g["prefill_packed"], what="packed conv", max_mismatch_frac=0.01)
    assert_bf16_close(G.depthwise_causal_conv4_prefill(g["x"][:3], g["weight"]), g["prefill_single"], what="single conv",
                      max_mismatch_frac=0.01)
    # [D,1,4] checkpoint layout of the weight and a row-strided input
    wide = torch.zeros(g["x"].shape[0], 8224, dtype=torch.bfloat16, device=DEV)
    wide[:, :6144] = g["x"]
    out3 = G.depthwise_causal_conv4_prefill(wide[:, :6144], g["weight"].unsqueeze(1), g["seq_start"])
    assert torch.equal(out3, out)
    state = g["state_garbage"].clone()
    G.conv_state_from_packed_prefill(state, g["x"], g["cu_seqlens"])
    assert torch.equal(state, g["state_from_packed"])
    assert torch.equal(G.conv_state_from_prefill(g["x"][:3]), g["state_from_prefill_short"])
    assert torch.equal(G.conv_weight_for_decode(g["weight"]), g["weight4"])
    st = g["decode_state_in"].clone()
    y = G.depthwise_causal_conv4_decode(g["decode_fused_row"][:, :6144], st, g["weight4"])
    assert torch.equal(st, g["decode_state_out"])
    assert_bf16_close(y, g["decode_out"], what="decode conv", max_mismatch_frac=0.01)


def test_norm_gate_gather_operators(mods, golden):
    _, G = mods
    g = dev(golden("glue_norms"))
    assert_bf16_close(G.qwen_rmsnorm(g["rms.x2"], g["rms.w1024"], 1e-6), g["rms.out2"], what="rmsnorm rows",
                      max_mismatch_frac=0.01)
    view = g["rms.fused"][:, :2048].view(3, 8, 256)
    out = G.qwen_rmsnorm(view, g["rms.w256"], 1e-6)
    assert out.is_contiguous()
    assert_bf16_close(out, g["rms.out3"], what="rmsnorm heads", max_mismatch_frac=0.01)
    t, h, d = 5, 16, 128
    conv, ab = g["qk.conv"], g["qk.ab"]
    q_n, k_n, beta, gg = G.gdn_qk_norm_gates(conv[:, : h * d].view(t, h, d), conv[:, h * d: 2 * h * d].view(t, h, d),
                                             ab[:, :h], ab[:, h:], g["qk.a_log"], g["qk.dt_bias"])
    assert q_n.is_contiguous() and k_n.is_contiguous()
    assert_bf16_close(q_n, g["qk.q_n"], what="q_n", max_mismatch_frac=0.01)
    assert_bf16_close(k_n, g["qk.k_n"], what="k_n", max_mismatch_frac=0.01)
    torch.testing.assert_close(beta, g["qk.beta"], rtol=5e-6, atol=1e-7)
    torch.testing.assert_close(gg, g["qk.g"], rtol=5e-6, atol=1e-7)
    z = g["gn.z_rows"][:, : h * d].view(t, h, d)
    assert_bf16_close(G.gdn_gated_rmsnorm(g["gn.x"], z, g["gn.weight"]), g["gn.out"], what="gated norm",
                      max_mismatch_frac=0.02)
    gu = g["swiglu.gate_up"]
    assert_bf16_close(G.swiglu(gu[:, :3584], gu[:, 3584:]), g["swiglu.out"], what="swiglu", max_mismatch_frac=0.02)
    assert_bf16_close(G.swiglu(gu[:, :3584].contiguous(), gu[:, 3584:].contiguous()), g["swiglu.out"], what="swiglu",
                      max_mismatch_frac=0.02)
    assert torch.equal(G.embedding_gather(g["gather.ids"], g["gather.table"]), g["gather.out"])
    assert torch.equal(G.embedding_gather(g["gather.ids"].long(), g["gather.table"]), g["gather.out"])
    a, b = g["rms.x2"], g["rms.out2"]
    assert torch.equal(G.residual_add(a, b), a + b)


def test_gemm_and_lm_head_operators(mods, golden):
    _, G = mods
    g = dev(golden("glue_matmul"))
    for m in (1, 5):
        assert_bf16_close(G.gemm_2d(g[f"gemm.x{m}"], g["gemm.w"]), g[f"gemm.y{m}"], what=f"gemm M={m}",
                          max_mismatch_frac=0.05)
    ids = G.lm_head_argmax(g["argmax.rows"], g["argmax.table"], last_only=False)
    assert ids.dtype == torch.int64 and torch.equal(ids, g["argmax.ids"])
    last = G.lm_head_argmax(g["argmax.rows"], g["argmax.table"], last_only=True)
    assert last.ndim == 0 and int(last) == int(g["argmax.last"])
    # more rows than one launch takes (32): served in slices
    rows = g["argmax.rows"].repeat(15, 1)[:40].contiguous()
    assert torch.equal(G.lm_head_argmax(rows, g["argmax.table"], last_only=False), g["argmax.ids"].repeat(15)[:40])


def test_gdn_decode_layer_kernels_against_reference_chain(mods, golden):
    """engine/runner.py:423-441 run with the reference's kernels vs (a) the drop-in chain, (b) prep + step + norm,
    (c) the one-launch mixer."""
    ops, G = mods
    g = dev(golden("glue_gdn_decode_layer"))
    batch, h, d = g["state_in"].shape[0], g["state_in"].shape[1], 128
    kd = h * d
    fused = g["fused"]

    def check(out, conv_state, state, tag):
        assert torch.equal(conv_state, g["conv_state_out"]), tag
        # a one-ulp flip of a bf16 conv output v[c] (different exp libraries) moves the whole state column c by
        # k * beta * ulp: columns either agree to fp32 rounding or differ by that much, and only a few of them do
        diff = (state - g["state_out"]).abs()
        assert diff.max().item() <= 2.0 ** -7 * 4.0, f"{tag} state: max abs {diff.max().item()}"
        touched = (diff.amax(dim=2) > 1e-5).float().mean().item()
        assert touched <= 0.02, f"{tag} state: {touched:.2%} of the columns differ"
        # the output went through two more roundings (q_n/k_n, core) on slightly different transcendentals
        assert_bf16_close(out, g["out"], ulps=2, what=tag, max_mismatch_frac=0.05)

    # (a) drop-in operator chain
    cs, st = g["conv_state_in"].clone(), g["state_in"].clone()
    conv = G.depthwise_causal_conv4_decode(fused[:, : 3 * kd], cs, g["weight4"])
    assert_bf16_close(conv, g["conv"], what="conv", max_mismatch_frac=0.01)
    q_n, k_n, beta, gg = G.gdn_qk_norm_gates(conv[:, :kd].view(batch, h, d), conv[:, kd: 2 * kd].view(batch, h, d),
                                             fused[:, 4 * kd: 4 * kd + h], fused[:, 4 * kd + h:], g["a_log"], g["dt_bias"])
    assert_bf16_close(q_n, g["q_n"], what="q_n", max_mismatch_frac=0.02)
    assert_bf16_close(k_n, g["k_n"], what="k_n", max_mismatch_frac=0.02)
    torch.testing.assert_close(gg, g["g"], rtol=5e-6, atol=1e-7)
    core = ops.gdn_recurrent_decode(q_n, k_n, conv[:, 2 * kd:].view(batch, h, d), beta, gg, st)
    out = G.gdn_gated_rmsnorm(core, fused[:, 3 * kd: 4 * kd].view(batch, h, d), g["norm_weight"])
    check(out.view(batch, kd), cs, st, "drop-in chain")
    # the recurrence alone on the reference's own intermediates: fp32 rounding only
    st = g["state_in"].clone()
    core = ops.gdn_recurrent_decode(g["q_n"], g["k_n"], g["conv"][:, 2 * kd:].view(batch, h, d), g["beta"], g["g"], st)
    torch.testing.assert_close(st, g["state_out"], rtol=1e-5, atol=1e-6)
    assert_bf16_close(core, g["core"], what="core", max_mismatch_frac=0.01)
    # (b) fused prep kernel + step + gated norm
    cs, st = g["conv_state_in"].clone(), g["state_in"].clone()
    q_n, k_n, v, beta, gg = ops.gdn_decode_prep(fused[:, : 3 * kd], cs, g["weight4"], fused[:, 4 * kd: 4 * kd + h],
                                                fused[:, 4 * kd + h:], g["a_log"], g["dt_bias"], h)
    assert_bf16_close(q_n, g["q_n"], what="prep q_n", max_mismatch_frac=0.02)
    assert_bf16_close(k_n, g["k_n"], what="prep k_n", max_mismatch_frac=0.02)
    torch.testing.assert_close(beta, g["beta"], rtol=5e-6, atol=1e-7)
    torch.testing.assert_close(gg, g["g"], rtol=1e-5, atol=1e-7)
    core = ops.gdn_recurrent_decode(q_n, k_n, v, beta, gg, st)
    out = ops.gdn_gated_rmsnorm_fused(core, fused[:, 3 * kd: 4 * kd], g["norm_weight"])
    check(out, cs, st, "prep + step + norm")
    # (c) the whole mixer in one launch
    for overlap in (0, ops.OVERLAP_START | ops.OVERLAP_PREFETCH):
        cs, st = g["conv_state_in"].clone(), g["state_in"].clone()
        out = ops.gdn_decode_fused(fused, cs, g["weight4"], g["a_log"], g["dt_bias"], g["norm_weight"], st, h,
                                   overlap=overlap)
        check(out, cs, st, f"one-launch mixer (overlap {overlap})")


def test_attention_decode_layer_against_reference_chain(mods, golden):
    """engine/runner.py:464-517 run with the reference's kernels vs the fused decode kernel with the q/k head norms
    inside, and vs the drop-in chain."""
    ops, G = mods
    g = dev(golden("glue_attn_decode_layer"))
    batch, hq, hkv, d = 3, 8, 2, 256
    qd, kvd = hq * d, hkv * d
    fused = g["fused"]
    q_raw = fused[:, :qd].view(batch, hq, d)
    k_raw = fused[:, 2 * qd: 2 * qd + kvd].view(batch, hkv, d)
    v_raw = fused[:, 2 * qd + kvd:].view(batch, hkv, d)
    gate = fused[:, qd: 2 * qd]
    ws = ops.fused_decode_workspace(DEV)

    def check(out, kc, vc, tag):
        assert torch.equal(vc, g["v_cache_out"]), tag
        assert_bf16_close(kc, g["k_cache_out"], what=f"{tag} k cache", max_mismatch_frac=0.001)
        err = (out.float() - g["out"].float()).abs().max().item()
        assert err <= 2.0 ** -6, f"{tag}: max abs {err}"

    for partition in (0, 1, 2, 3):
        kc, vc = g["k_cache_in"].clone(), g["v_cache_in"].clone()
        out = ops.fused_decode_attention(q_raw, k_raw, v_raw, gate, kc, vc, g["block_table"], g["pos"], g["inv_freq"], 64,
                                         ws, q_norm_weight=g["q_norm_weight"], k_norm_weight=g["k_norm_weight"],
                                         eps=1e-6, partition=partition)
        check(out, kc, vc, f"fused, norms inside, partition {partition}")
    # drop-in chain through the registered operators
    kc, vc = g["k_cache_in"].clone(), g["v_cache_in"].clone()
    q = G.qwen_rmsnorm(q_raw, g["q_norm_weight"], 1e-6)
    k = G.qwen_rmsnorm(k_raw, g["k_norm_weight"], 1e-6)
    assert_bf16_close(q, g["q_normed"], what="q norm", max_mismatch_frac=0.01)
    assert_bf16_close(k, g["k_normed"], what="k norm", max_mismatch_frac=0.01)
    ids = g["pos"].view(batch, 1)
    q4 = ops.partial_rope(q.unsqueeze(2), ids, g["inv_freq"], 64)
    k4 = ops.partial_rope(k.unsqueeze(2), ids, g["inv_freq"], 64)
    ctx = ops.call_paged_gqa_attention_decode_triton(q4[:, :, 0, :].contiguous(), k4[:, :, 0, :].contiguous(),
                                                     v_raw.contiguous(), kc, vc, g["block_table"], g["pos"])
    assert (ctx.float() - g["ctx"].float()).abs().max().item() <= 2.0 ** -6
    gate4 = gate.reshape(batch, hq, d).permute(1, 0, 2).unsqueeze(0).contiguous()
    out = ops.attention_gate_pack(ctx.permute(1, 0, 2).unsqueeze(0).contiguous(), gate4)
    check(out, kc, vc, "drop-in chain")
    torch.cuda.synchronize()
    import b200attn
    assert b200attn.load().b200_wait_timed_out() == 0


def test_single_sequence_baselines(mods):
    """The runner's two single-sequence operators served by the path kernels: fixed-length causal prefill equals the
    packed varlen operator; contiguous-cache decode equals the paged chain over the same tokens."""
    ops, G = mods
    gen = torch.Generator().manual_seed(31)
    t = 70
    q_thd = torch.randn(t, 8, 256, generator=gen).to(torch.bfloat16).to(DEV)
    k_thd = torch.randn(t, 2, 256, generator=gen).to(torch.bfloat16).to(DEV)
    v_thd = torch.randn(t, 2, 256, generator=gen).to(torch.bfloat16).to(DEV)
    cu, max_len = ops.build_cu_seqlens([t], device=DEV)
    ref = ops.gqa_attention_varlen_causal(q_thd, k_thd, v_thd, cu, max_len)
    q4, k4, v4 = (x.unsqueeze(0).permute(0, 2, 1, 3) for x in (q_thd, k_thd, v_thd))   # [1,H,T,D] views
    out = G.gqa_attention_without_kvcache_casual(q4, k4, v4)
    assert out.shape == q4.shape
    assert torch.equal(out[0].permute(1, 0, 2), ref)
    # contiguous cache of 100 tokens (not a multiple of 16), 70 cached, append one more
    kc, vc = G.allocate_kv_cache(2, 100, 256, device=DEV)
    assert kc.shape == (2, 100, 256)
    kc[:, :t] = k_thd.permute(1, 0, 2)
    vc[:, :t] = v_thd.permute(1, 0, 2)
    qn = torch.randn(8, 256, generator=gen).to(torch.bfloat16).to(DEV)
    kn = torch.randn(2, 256, generator=gen).to(torch.bfloat16).to(DEV)
    vn = torch.randn(2, 256, generator=gen).to(torch.bfloat16).to(DEV)
    pos = torch.tensor([t], dtype=torch.int64, device=DEV)
    got = G.call_gqa_attention_decode_split_triton(qn, kn, vn, kc, vc, pos)
    assert got.shape == (8, 256)
    assert torch.equal(kc[:, t], kn) and torch.equal(vc[:, t], vn)
    # the same tokens in a paged cache
    pk, pv = ops.allocate_paged_kv_cache(8, 2, 256, device=DEV)
    table = torch.tensor([[5, 2, 7, 0, 3]], dtype=torch.int32, device=DEV)
    ops.paged_kv_fill(pk, pv, k_thd.permute(1, 0, 2), v_thd.permute(1, 0, 2), table[0])
    want = ops.call_paged_gqa_attention_decode_triton(qn[None], kn[None], vn[None], pk, pv, table, pos)
    assert torch.equal(got, want[0])
    # a cache whose storage ends inside its last page is refused before any launch
    tight = torch.zeros(2, 100, 256, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(AssertionError):
        G.call_gqa_attention_decode_split_triton(qn, kn, vn, tight, tight.clone(), pos)
