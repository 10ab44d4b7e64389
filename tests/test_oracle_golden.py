"""Pins the CPU oracle against outputs of the REFERENCE operators (tests/golden/*.pt, made by
tests/golden/make_golden.py with the reference's Triton kernels under the interpreter)."""
import torch

from oracle import reference_ops as O


def maxabs(a, b):
    return (a.float() - b.float()).abs().max().item()


def test_paged_decode_cfg1(golden):
    g = golden("paged_decode_cfg1")
    kc, vc = g["k_cache_in"].clone(), g["v_cache_in"].clone()
    b, hq, d = g["q"].shape
    m = torch.full((b, hq, O.MAX_SPLITS), 7.0)
    l = torch.full((b, hq, O.MAX_SPLITS), 3.0)
    acc = torch.full((b, hq, O.MAX_SPLITS, d), -5.0)
    out = O.paged_decode(g["q"], g["k_new"], g["v_new"], kc, vc, g["block_table"], g["pos"], (m, l, acc))
    assert torch.equal(kc, g["k_cache_out"]) and torch.equal(vc, g["v_cache_out"])  # bit-exact
    keep = int(g["partial_keep"])
    assert torch.equal(torch.isinf(m[:, :, :keep]), torch.isinf(g["m_partial_head"]))
    fin = ~torch.isinf(m[:, :, :keep])
    assert maxabs(m[:, :, :keep][fin], g["m_partial_head"][fin]) < 1e-5
    assert maxabs(l[:, :, :keep], g["l_partial_head"]) < 1e-4
    assert maxabs(acc[:, :, :keep], g["acc_partial_head"]) < 1e-4
    assert torch.isinf(m[:, :, keep:]).all() and (l[:, :, keep:] == 0).all() and (acc[:, :, keep:] == 0).all()
    assert maxabs(out, g["out"]) <= 2 ** -8  # at most one bf16 ulp at |x|<=1
    # reference's own torch function and ours agree, and sit within the 2e-2 bar of the kernel
    exact = O.paged_decode_exact(g["q"], kc, vc, g["block_table"], (g["pos"] + 1).tolist())
    assert maxabs(exact.to(torch.bfloat16), g["out_torch_ref"]) <= 2 ** -8
    assert maxabs(exact, g["out"]) < 2e-2


def test_paged_fill_varlen(golden):
    g = golden("paged_fill_varlen")
    for tag in ("a", "b"):
        kc, vc = g[f"{tag}.k_cache_in"].clone(), g[f"{tag}.v_cache_in"].clone()
        O.paged_kv_fill_varlen(kc, vc, g[f"{tag}.k_thd"].permute(1, 0, 2), g[f"{tag}.v_thd"].permute(1, 0, 2),
                               g[f"{tag}.block_table"], g[f"{tag}.cu_seqlens"])
        assert torch.equal(kc, g[f"{tag}.k_cache_out"]) and torch.equal(vc, g[f"{tag}.v_cache_out"])


def test_varlen_causal(golden):
    g = golden("varlen_causal")
    out = O.varlen_causal(g["q"], g["k"], g["v"], g["cu_seqlens"], int(g["tile_kv"]), int(g["block_q"]))
    assert maxabs(out, g["out"]) <= 2 ** -6
    assert (out.float() - g["out"].float()).abs().mean().item() < 1e-4
    exact = O.varlen_causal_exact(g["q"], g["k"], g["v"], g["cu_seqlens"])
    assert maxabs(exact.to(torch.bfloat16), g["out_torch_ref"]) <= 2 ** -7
    assert maxabs(exact, g["out"]) < 2e-2 * max(1.0, exact.abs().max().item())


def test_partial_rope(golden):
    g = golden("partial_rope")
    out = O.partial_rope(g["a.x"], g["a.ids"], g["a.inv_freq"], int(g["a.rotary_dim"]))
    assert maxabs(out, g["a.out"]) <= 2 ** -6
    assert torch.equal(out[..., 64:], g["a.out"][..., 64:])
    xb = g["b.x_thd"].unsqueeze(0).permute(0, 2, 1, 3)
    out = O.partial_rope(xb, g["b.ids"], g["a.inv_freq"], 64)
    assert maxabs(out, g["b.out"]) <= 2 ** -6
    out = O.partial_rope(g["c.x"], g["c.ids"], g["c.inv_freq"], int(g["c.rotary_dim"]))
    assert maxabs(out, g["c.out"]) <= 2 ** -6
    assert torch.equal(out[..., 96:], g["c.out"][..., 96:])


def test_gate_pack(golden):
    g = golden("gate_pack")
    t, h, d = g["ctx_thd"].shape
    x4 = g["ctx_thd"].permute(1, 0, 2).unsqueeze(0)
    g4 = g["gate"].view(1, t, h, d).permute(0, 2, 1, 3)
    out = O.attention_gate_pack(x4, g4)
    assert out.shape == g["out"].shape
    assert maxabs(out, g["out"]) <= 2 ** -7


def test_gdn_decode(golden):
    g = golden("gdn_decode")
    state = g["state_in"].clone()
    out = O.gdn_recurrent_decode(g["q"], g["k"], g["v"], g["beta"], g["g"], state)
    assert maxabs(out, g["out"]) <= 2 ** -8
    assert maxabs(state, g["state_out"]) < 1e-6


def test_gdn_sequential(golden):
    g = golden("gdn_sequential")
    out, state = O.gdn_recurrent_prefill_sequential(g["q"], g["k"], g["v"], g["beta"], g["g"], g["cu_seqlens"])
    assert maxabs(out, g["out"]) <= 2 ** -8
    assert maxabs(state, g["state"]) < 1e-6
    out1, state1 = O.gdn_recurrent_prefill_sequential(g["q"][:4], g["k"][:4], g["v"][:4], g["beta"][:4], g["g"][:4])
    assert state1.shape == state.shape[1:] and torch.equal(state1, state[0])


def test_gdn_chunked(golden):
    g = golden("gdn_chunked")
    w, u, gcs = O.gdn_chunk_prepare_wy(g["k"], g["v"], g["beta"], g["g"])
    assert maxabs(gcs, g["g_cumsum"]) < 2e-6 * g["g_cumsum"].abs().max().item()  # fp32 prefix-sum order
    assert maxabs(w, g["w"]) < 2e-4 and maxabs(u, g["u_base"]) < 2e-4
    delta, cs, fs = O.gdn_chunk_state(g["k"], g["w"], g["u_base"], g["g_cumsum"])
    assert maxabs(delta, g["delta"]) < 2e-4
    assert maxabs(cs, g["chunk_state"]) < 2e-4 and maxabs(fs, g["final_state"]) < 2e-4
    out = O.gdn_chunk_output(g["q"], g["k"], g["delta"], g["g_cumsum"], g["chunk_state"])
    assert maxabs(out, g["out"]) <= 1e-2
    # end to end against the token-serial recurrence (the reference's own acceptance bars)
    out2, fs2 = O.gdn_chunked_prefill(g["q"], g["k"], g["v"], g["beta"], g["g"])
    assert maxabs(out2, g["seq_out"]) < 1e-2 and maxabs(fs2, g["seq_state"]) < 5e-4
