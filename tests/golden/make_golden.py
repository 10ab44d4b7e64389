"""Generate the golden vectors under tests/golden/ by running the REFERENCE operators.

Usage (CPU only, needs the reference checkout; it is never needed at test time):

    python tests/golden/make_golden.py --reference <path-to-reference-checkout>

The reference operators are Triton kernels.  They are executed here on the CPU with
``TRITON_INTERPRET=1`` plus four harness-side shims (the reference files are not modified):

1. every ``triton.runtime.autotuner.Autotuner`` is pinned to its first config, because the
   autotuner benchmarks on a GPU driver that does not exist on a CPU box;
2. ``InterpreterBuilder.create_dot`` is replaced by a version that widens bf16 operands to fp32
   (the stock Triton 3.6 interpreter multiplies the raw uint16 bit patterns);
3. ``torch.library.wrap_triton`` passes ``InterpretedFunction`` objects through (two GDN chunk
   kernels have no autotune wrapper and would otherwise be rejected);
4. ``InterpreterBuilder.cast_impl`` rounds fp32 -> bf16 to nearest-even, as the GPU's ``cvt.rn.bf16.f32``
   does for ``.to(tl.bfloat16)`` and for stores through a bf16 pointer (the stock interpreter truncates).

Each case stores the seeded inputs AND the reference outputs, so the tests need neither the
reference nor Triton.  Everything is small (the interpreter runs one Python program per CTA).
"""
from __future__ import annotations

import argparse
import os
import sys
import time
from pathlib import Path

os.environ["TRITON_INTERPRET"] = "1"

import numpy as np  # noqa: E402
import torch  # noqa: E402

HERE = Path(__file__).resolve().parent


# --------------------------------------------------------------------------- shims
def install_shims():
    """The four interpreter shims live in baseline/interpreter_shims.py (shared with the CPU-baseline harness)."""
    import importlib.util
    path = HERE.parent.parent / "baseline" / "interpreter_shims.py"
    spec = importlib.util.spec_from_file_location("interpreter_shims", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.install_shims()


# --------------------------------------------------------------------------- inputs
def bf16_randn(*shape, gen):
    return torch.randn(*shape, generator=gen, dtype=torch.float32).to(torch.bfloat16)


def gdn_inputs(token_num, heads, dk, dv, gen, v_row_stride=None):
    """q/k L2-normalised per head (q also times dk**-0.5) then rounded to bf16; beta in (0,1);
    g = -softplus(N(0,1)) * exp(A), A ~ U(0, 2.7) per head."""
    q = torch.randn(token_num, heads, dk, generator=gen)
    k = torch.randn(token_num, heads, dk, generator=gen)
    q = (q * torch.rsqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dk**-0.5).to(torch.bfloat16)
    k = (k * torch.rsqrt((k * k).sum(-1, keepdim=True) + 1e-6)).to(torch.bfloat16)
    if v_row_stride is None:
        v = bf16_randn(token_num, heads, dv, gen=gen)
    else:  # a [T, H, DV] view into a wider row, like the runner's slice of the conv output
        storage = bf16_randn(token_num, v_row_stride, gen=gen)
        v = storage[:, v_row_stride - heads * dv:].view(token_num, heads, dv)
    beta = torch.sigmoid(torch.randn(token_num, heads, generator=gen))
    a = torch.rand(heads, generator=gen) * 2.7
    g = -torch.nn.functional.softplus(torch.randn(token_num, heads, generator=gen)) * torch.exp(a)
    return q, k, v, beta, g


def shuffled_table(batch, pages_per_seq, num_pages, gen):
    order = torch.randperm(num_pages, generator=gen)
    return order[: batch * pages_per_seq].view(batch, pages_per_seq).to(torch.int32).contiguous()


# --------------------------------------------------------------------------- cases
def case_paged_decode_cfg1():
    """B=4, contexts [37,64,100,128], 8 Q heads / 2 KV heads / D=256, page 16, seed 0."""
    from triton_kernels import gqa_attention_decode_paged as ref

    gen = torch.Generator().manual_seed(0)
    lens = [37, 64, 100, 128]
    batch, hq, hkv, d = 4, 8, 2, 256
    pps = (128 + 15) // 16 + 1
    num_pages = batch * pps
    block_table = shuffled_table(batch, pps, num_pages, gen)
    k_cache = bf16_randn(num_pages, hkv, 16, d, gen=gen)
    v_cache = bf16_randn(num_pages, hkv, 16, d, gen=gen)
    q = bf16_randn(batch, hq, d, gen=gen)
    k_new = bf16_randn(batch, hkv, d, gen=gen)
    v_new = bf16_randn(batch, hkv, d, gen=gen)
    pos = torch.tensor([n - 1 for n in lens], dtype=torch.int64)

    kc, vc = k_cache.clone(), v_cache.clone()
    # dirty scratch on purpose: stale partials must not leak into the result
    m = torch.full((batch, hq, ref.MAX_SPLITS), 7.0)
    l = torch.full((batch, hq, ref.MAX_SPLITS), 3.0)
    acc = torch.full((batch, hq, ref.MAX_SPLITS, d), -5.0)
    out = ref.call_paged_gqa_attention_decode_triton(
        q, k_new, v_new, kc, vc, block_table, pos, (m, l, acc)
    )
    keep = 16  # only the first cdiv(128,16)=8 splits can be active; the rest must be (-inf,0,0)
    assert torch.isinf(m[:, :, keep:]).all() and (l[:, :, keep:] == 0).all()
    assert (acc[:, :, keep:] == 0).all()
    return dict(
        q=q, k_new=k_new, v_new=v_new, k_cache_in=k_cache, v_cache_in=v_cache,
        block_table=block_table, pos=pos,
        k_cache_out=kc, v_cache_out=vc,
        m_partial_head=m[:, :, :keep].clone(), l_partial_head=l[:, :, :keep].clone(),
        acc_partial_head=acc[:, :, :keep].clone(), partial_keep=torch.tensor(keep),
        out=out,
        out_torch_ref=ref.torch_paged_reference(q, kc, vc, block_table, lens),
    )


def case_paged_fill_varlen():
    from triton_kernels import gqa_attention_decode_paged as ref

    gen = torch.Generator().manual_seed(11)
    out = {}
    for tag, lengths in (("a", [7, 100, 1, 64]), ("b", [16, 17, 1])):
        batch, total = len(lengths), sum(lengths)
        hkv, d = 2, 256
        pps = (max(lengths) + 15) // 16
        num_pages = batch * pps + 8
        order = torch.randperm(num_pages, generator=gen)
        block_table = order[: batch * pps].view(batch, pps).to(torch.int32).contiguous()
        cu = torch.tensor([0] + list(np.cumsum(lengths)), dtype=torch.int32)
        # [T, H, D] storage viewed as [H, T, D]: the permuted views the runner passes
        k_thd = bf16_randn(total, hkv, d, gen=gen)
        v_thd = bf16_randn(total, hkv, d, gen=gen)
        init_k = bf16_randn(num_pages, hkv, 16, d, gen=gen)
        init_v = bf16_randn(num_pages, hkv, 16, d, gen=gen)
        kc, vc = init_k.clone(), init_v.clone()
        ref.paged_kv_fill_varlen(
            kc, vc, k_thd.permute(1, 0, 2), v_thd.permute(1, 0, 2), block_table, cu, max(lengths)
        )
        kr, vr = init_k.clone(), init_v.clone()
        ref.paged_kv_fill_varlen_torch(
            kr, vr, k_thd.permute(1, 0, 2), v_thd.permute(1, 0, 2), block_table, cu
        )
        assert torch.equal(kc, kr) and torch.equal(vc, vr)
        out.update({
            f"{tag}.lengths": torch.tensor(lengths), f"{tag}.block_table": block_table,
            f"{tag}.cu_seqlens": cu, f"{tag}.k_thd": k_thd, f"{tag}.v_thd": v_thd,
            f"{tag}.k_cache_in": init_k, f"{tag}.v_cache_in": init_v,
            f"{tag}.k_cache_out": kc, f"{tag}.v_cache_out": vc,
        })
    return out


def case_varlen_causal():
    from triton_kernels import gqa_attention_varlen_causal as ref

    gen = torch.Generator().manual_seed(2)
    lengths = [1, 3, 17, 64, 40]
    total = sum(lengths)
    q = bf16_randn(total, 8, 256, gen=gen)
    k = bf16_randn(total, 2, 256, gen=gen)
    v = bf16_randn(total, 2, 256, gen=gen)
    cu, max_len = ref.build_cu_seqlens(lengths, device="cpu")
    out = ref.gqa_attention_varlen_causal(q, k, v, cu, max_len)
    cfg = ref._gqa_attention_varlen_causal_triton.configs[0]
    return dict(
        lengths=torch.tensor(lengths), cu_seqlens=cu, q=q, k=k, v=v, out=out,
        out_torch_ref=ref.torch_varlen_reference(q, k, v, lengths),
        tile_kv=torch.tensor(cfg.kwargs["TILE_KV_S"]), block_q=torch.tensor(cfg.kwargs["BLOCK_Q_S"]),
    )


def case_partial_rope():
    from triton_kernels import partial_rope as ref

    gen = torch.Generator().manual_seed(5)
    out = {}
    # (a) model shape, decode-like layout [B,H,1,D] with large positions, int64 ids
    r, d = 64, 256
    inv_freq = (1.0 / (1e7 ** (torch.arange(0, r, 2, dtype=torch.float32) / r))).contiguous()
    x = bf16_randn(3, 8, 1, d, gen=gen)
    ids = torch.tensor([[0], [4095], [32768]], dtype=torch.int64)
    out.update({"a.x": x, "a.ids": ids, "a.inv_freq": inv_freq, "a.rotary_dim": torch.tensor(r),
                "a.out": ref.partial_rope(x, ids, inv_freq, r)})
    # (b) prefill-like: [1,H,T,D] as a permuted view of [T,H,D], int32 ids restarting per sequence
    t = 21
    x_thd = bf16_randn(t, 2, d, gen=gen)
    xb = x_thd.unsqueeze(0).permute(0, 2, 1, 3)
    ids = torch.cat([torch.arange(13), torch.arange(8)]).to(torch.int32).unsqueeze(0)
    out.update({"b.x_thd": x_thd, "b.ids": ids, "b.out": ref.partial_rope(xb, ids, inv_freq, r)})
    # (c) non-power-of-two rotary and head dims
    r2, d2 = 96, 160
    inv2 = (1.0 / (1e4 ** (torch.arange(0, r2, 2, dtype=torch.float32) / r2))).contiguous()
    xc = bf16_randn(2, 3, 5, d2, gen=gen)
    idc = torch.randint(0, 1000, (2, 5), generator=gen, dtype=torch.int64)
    out.update({"c.x": xc, "c.ids": idc, "c.inv_freq": inv2, "c.rotary_dim": torch.tensor(r2),
                "c.out": ref.partial_rope(xc, idc, inv2, r2)})
    return out


def case_gate_pack():
    from triton_kernels import attention_gate_pack as ref

    gen = torch.Generator().manual_seed(6)
    t, h, d = 5, 8, 256
    ctx_thd = bf16_randn(t, h, d, gen=gen)      # attention output [T,H,D]
    gate_t = bf16_randn(t, h * d, gen=gen)      # gate projection [T, H*D]
    x4 = ctx_thd.permute(1, 0, 2).unsqueeze(0)
    g4 = gate_t.view(1, t, h, d).permute(0, 2, 1, 3)
    return dict(ctx_thd=ctx_thd, gate=gate_t, out=ref.attention_gate_pack(x4, g4))


def case_gdn_decode():
    from triton_kernels import gdn_recurrent_prefill as ref

    gen = torch.Generator().manual_seed(3)
    batch, heads, dk, dv = 3, 4, 128, 128
    q, k, v, beta, g = gdn_inputs(batch, heads, dk, dv, gen, v_row_stride=3 * heads * dv)
    state = torch.randn(batch, heads, dk, dv, generator=gen) * 0.1
    s = state.clone()
    out = ref.gdn_recurrent_decode(q, k, v, beta, g, s)
    return dict(q=q, k=k, v=v.contiguous(), beta=beta, g=g, state_in=state, state_out=s, out=out)


def case_gdn_sequential():
    from triton_kernels import gdn_recurrent_prefill as ref

    gen = torch.Generator().manual_seed(4)
    heads, dk, dv = 2, 128, 128
    lengths = [4, 1, 6]
    total = sum(lengths)
    q, k, v, beta, g = gdn_inputs(total, heads, dk, dv, gen)
    cu = torch.tensor([0] + list(np.cumsum(lengths)), dtype=torch.int32)
    out, state = ref.gdn_recurrent_prefill_sequential(q, k, v, beta, g, cu)
    out1, state1 = ref.gdn_recurrent_prefill_sequential(q[:4], k[:4], v[:4], beta[:4], g[:4])
    assert torch.equal(out1, out[:4]) and torch.equal(state1, state[0])
    return dict(q=q, k=k, v=v, beta=beta, g=g, cu_seqlens=cu, out=out, state=state)


def case_gdn_chunked():
    from triton_kernels import gdn_recurrent_prefill as ref

    gen = torch.Generator().manual_seed(7)
    heads, dk, dv = 2, 128, 128
    total = 130  # two full chunks + a ragged third
    q, k, v, beta, g = gdn_inputs(total, heads, dk, dv, gen)
    w, u_base, g_cumsum = ref.gdn_chunk_prepare_wy(k, v, beta, g)
    delta, chunk_state, final_state = ref.gdn_chunk_state(k, w, u_base, g_cumsum)
    out = ref.gdn_chunk_output(q, k, delta, g_cumsum, chunk_state)
    seq_out, seq_state = ref._torch_sequential_reference(q, k, v, beta, g)
    return dict(q=q, k=k, v=v, beta=beta, g=g, w=w, u_base=u_base, g_cumsum=g_cumsum,
                delta=delta, chunk_state=chunk_state, final_state=final_state, out=out,
                seq_out=seq_out, seq_state=seq_state)


def case_glue_conv4():
    """Depthwise conv4: packed prefill with seq_start, single-token decode with a non-zero state, conv-state extraction."""
    from triton_kernels import depthwise_causal_conv4_decode as dec
    from triton_kernels import depthwise_causal_conv4_prefill as pre

    gen = torch.Generator().manual_seed(21)
    chans = 6144
    lengths = [3, 6, 2]
    total = sum(lengths)
    x = bf16_randn(total, chans, gen=gen)
    w = (torch.randn(chans, 4, generator=gen) * 0.5).to(torch.bfloat16)
    seq_start = pre.build_seq_start(lengths, device="cpu")
    cu = torch.tensor([0] + list(np.cumsum(lengths)), dtype=torch.int32)
    out = {"lengths": torch.tensor(lengths), "x": x, "weight": w, "seq_start": seq_start, "cu_seqlens": cu,
           "prefill_packed": pre.depthwise_causal_conv4_prefill(x, w, seq_start),
           "prefill_single": pre.depthwise_causal_conv4_prefill(x[:3], w)}
    state = bf16_randn(len(lengths), 4, chans, gen=gen)      # non-zero on purpose: every slot must be overwritten
    out["state_garbage"] = state.clone()
    dec.conv_state_from_packed_prefill(state, x, cu)
    out["state_from_packed"] = state.clone()
    out["state_from_prefill_short"] = dec.conv_state_from_prefill(x[:3])
    # decode: x is a column slice of a wider projection row, as in the runner
    batch = 3
    fused = bf16_randn(batch, 8224, gen=gen)
    w4 = dec.conv_weight_for_decode(w)
    st = bf16_randn(batch, 4, chans, gen=gen)
    out.update({"decode_fused_row": fused, "decode_state_in": st.clone(), "weight4": w4})
    out["decode_out"] = dec.depthwise_causal_conv4_decode(fused[:, :chans], st, w4)
    out["decode_state_out"] = st
    return out


def case_glue_norms():
    """RMSNorm (flat rows and a [B,H,D] column view), q/k L2 norms + gates, gated RMSNorm, SwiGLU, gather."""
    from triton_kernels import embedding_gather as eg
    from triton_kernels import gdn_gated_rmsnorm as gn
    from triton_kernels import gdn_qk_norm_gates as qk
    from triton_kernels import qwen_rmsnorm as rn
    from triton_kernels import swiglu as sw

    gen = torch.Generator().manual_seed(22)
    out = {}
    x2 = bf16_randn(5, 1024, gen=gen)
    w1024 = (torch.randn(1024, generator=gen) * 0.1).to(torch.bfloat16)
    out.update({"rms.x2": x2, "rms.w1024": w1024, "rms.out2": rn.qwen_rmsnorm(x2, w1024, 1e-6)})
    fused = bf16_randn(3, 5120, gen=gen)
    w256 = (torch.randn(256, generator=gen) * 0.1).to(torch.bfloat16)
    out.update({"rms.fused": fused, "rms.w256": w256,
                "rms.out3": rn.qwen_rmsnorm(fused[:, :2048].view(3, 8, 256), w256, 1e-6)})
    # q/k norms + gates on strided views of a conv output, a/b as column slices
    t, h, d = 5, 16, 128
    conv = bf16_randn(t, 3 * h * d, gen=gen)
    ab = bf16_randn(t, 2 * h, gen=gen)
    a_log = torch.rand(h, generator=gen) * 2.7
    dt_bias = bf16_randn(h, gen=gen)
    q = conv[:, : h * d].view(t, h, d)
    k = conv[:, h * d: 2 * h * d].view(t, h, d)
    q_n, k_n, beta, g = qk.gdn_qk_norm_gates(q, k, ab[:, :h], ab[:, h:], a_log, dt_bias)
    out.update({"qk.conv": conv, "qk.ab": ab, "qk.a_log": a_log, "qk.dt_bias": dt_bias, "qk.q_n": q_n, "qk.k_n": k_n,
                "qk.beta": beta, "qk.g": g})
    core = bf16_randn(t, h, d, gen=gen)
    z = bf16_randn(t, h * d + 64, gen=gen)
    wn = 1.0 + torch.randn(d, generator=gen) * 0.1
    out.update({"gn.x": core, "gn.z_rows": z, "gn.weight": wn,
                "gn.out": gn.gdn_gated_rmsnorm(core, z[:, : h * d].view(t, h, d), wn)})
    inter = 3584
    gate_up = bf16_randn(3, 2 * inter, gen=gen)
    out.update({"swiglu.gate_up": gate_up, "swiglu.out": sw.swiglu(gate_up[:, :inter], gate_up[:, inter:])})
    table = bf16_randn(50, 1024, gen=gen)
    ids = torch.tensor([7, 0, 49, 7, 13], dtype=torch.int32)
    out.update({"gather.table": table, "gather.ids": ids, "gather.out": eg.embedding_gather(ids, table)})
    return out


def case_glue_matmul():
    """Projection GEMM and the fused LM-head arg-max (with a tie: two identical vocabulary rows)."""
    from triton_kernels import gemm_2d as gm
    from triton_kernels import vocab_argmax as va

    gen = torch.Generator().manual_seed(23)
    out = {}
    w = (torch.randn(384, 256, generator=gen) * 0.05).to(torch.bfloat16)
    for m in (1, 5):
        x = bf16_randn(m, 256, gen=gen)
        y = gm.gemm_2d(x, w)
        assert (y.float() - x.float() @ w.float().t()).abs().max() < 0.05
        out.update({f"gemm.x{m}": x, f"gemm.y{m}": y})
    out["gemm.w"] = w
    vocab, hidden = 2048, 256
    table = (torch.randn(vocab, hidden, generator=gen) * 0.05).to(torch.bfloat16)
    rows = bf16_randn(3, hidden, gen=gen)
    best = torch.argmax(rows.float() @ table.float().t(), dim=-1)
    table[1900] = table[best[0]]          # a later duplicate of row 0's winner: the lower index must still win
    table[3] = table[best[1]] if best[1] > 3 else table[3]
    ids_all = va.lm_head_argmax(rows, table, last_only=False)
    ids_last = va.lm_head_argmax(rows, table, last_only=True)
    ref = torch.argmax(rows.float() @ table.float().t(), dim=-1)
    assert torch.equal(ids_all, ref), (ids_all, ref)
    out.update({"argmax.rows": rows, "argmax.table": table, "argmax.ids": ids_all, "argmax.last": ids_last})
    return out


def case_glue_gdn_decode_layer():
    """The Gated-DeltaNet mixer of one decode token between its projections, as the reference runner chains it
    (engine/runner.py:423-441): conv4 decode -> q/k norms + gates -> delta-rule step -> gated RMSNorm."""
    from triton_kernels import depthwise_causal_conv4_decode as dec
    from triton_kernels import gdn_gated_rmsnorm as gn
    from triton_kernels import gdn_qk_norm_gates as qk
    from triton_kernels import gdn_recurrent_prefill as rec

    gen = torch.Generator().manual_seed(24)
    batch, h, d = 3, 4, 128
    kd = h * d
    fused = bf16_randn(batch, 4 * kd + 2 * h, gen=gen)
    conv_state = bf16_randn(batch, 4, 3 * kd, gen=gen)
    w4 = (torch.randn(4, 3 * kd, generator=gen) * 0.5).to(torch.bfloat16)
    a_log = torch.rand(h, generator=gen) * 2.7
    dt_bias = bf16_randn(h, gen=gen)
    norm_w = 1.0 + torch.randn(d, generator=gen) * 0.1
    state = torch.randn(batch, h, d, d, generator=gen) * 0.1
    cs, st = conv_state.clone(), state.clone()
    conv = dec.depthwise_causal_conv4_decode(fused[:, : 3 * kd], cs, w4)
    q = conv[:, :kd].view(batch, h, d)
    k = conv[:, kd: 2 * kd].view(batch, h, d)
    v = conv[:, 2 * kd:].view(batch, h, d)
    q_n, k_n, beta, g = qk.gdn_qk_norm_gates(q, k, fused[:, 4 * kd: 4 * kd + h], fused[:, 4 * kd + h:], a_log, dt_bias)
    core = rec.gdn_recurrent_decode(q_n, k_n, v, beta, g, st)
    normed = gn.gdn_gated_rmsnorm(core, fused[:, 3 * kd: 4 * kd].view(batch, h, d), norm_w)
    return dict(fused=fused, conv_state_in=conv_state, weight4=w4, a_log=a_log, dt_bias=dt_bias, norm_weight=norm_w,
                state_in=state, conv=conv, q_n=q_n, k_n=k_n, beta=beta, g=g, core=core, conv_state_out=cs,
                state_out=st, out=normed.view(batch, kd))


def case_glue_attn_decode_layer():
    """The attention mixer of one decode token between its projections, as the reference runner chains it
    (engine/runner.py:464-517): q/k RMSNorm -> partial RoPE -> append + paged attention -> sigmoid gate."""
    from triton_kernels import attention_gate_pack as gp
    from triton_kernels import gqa_attention_decode_paged as pa
    from triton_kernels import partial_rope as pr
    from triton_kernels import qwen_rmsnorm as rn

    gen = torch.Generator().manual_seed(25)
    lens = [5, 37, 100]
    batch, hq, hkv, d, r = len(lens), 8, 2, 256, 64
    qd, kvd = hq * d, hkv * d
    fused = bf16_randn(batch, 2 * qd + 2 * kvd, gen=gen)
    q_w = (torch.randn(d, generator=gen) * 0.1).to(torch.bfloat16)
    k_w = (torch.randn(d, generator=gen) * 0.1).to(torch.bfloat16)
    inv_freq = (1.0 / (1e7 ** (torch.arange(0, r, 2, dtype=torch.float32) / r))).contiguous()
    pps = (max(lens) + 1 + 15) // 16
    num_pages = batch * pps + 3
    block_table = shuffled_table(batch, pps, num_pages, gen)
    k_cache = bf16_randn(num_pages, hkv, 16, d, gen=gen)
    v_cache = bf16_randn(num_pages, hkv, 16, d, gen=gen)
    pos = torch.tensor(lens, dtype=torch.int64)
    kc, vc = k_cache.clone(), v_cache.clone()
    q = rn.qwen_rmsnorm(fused[:, :qd].view(batch, hq, d), q_w, 1e-6)
    k = rn.qwen_rmsnorm(fused[:, 2 * qd: 2 * qd + kvd].view(batch, hkv, d), k_w, 1e-6)
    ids = pos.view(batch, 1)
    q4 = pr.partial_rope(q.unsqueeze(2), ids, inv_freq, r)
    k4 = pr.partial_rope(k.unsqueeze(2), ids, inv_freq, r)
    v_new = fused[:, 2 * qd + kvd:].view(batch, hkv, d).contiguous()
    ctx = pa.call_paged_gqa_attention_decode_triton(q4[:, :, 0, :].contiguous(), k4[:, :, 0, :].contiguous(), v_new, kc, vc,
                                                    block_table, pos)
    gate4 = fused[:, qd: 2 * qd].view(batch, hq, d).permute(1, 0, 2).unsqueeze(0).contiguous()
    out = gp.attention_gate_pack(ctx.permute(1, 0, 2).unsqueeze(0).contiguous(), gate4)
    return dict(fused=fused, q_norm_weight=q_w, k_norm_weight=k_w, inv_freq=inv_freq, block_table=block_table,
                k_cache_in=k_cache, v_cache_in=v_cache, pos=pos, k_cache_out=kc, v_cache_out=vc, q_normed=q,
                k_normed=k, ctx=ctx, out=out)


CASES = {
    "paged_decode_cfg1": case_paged_decode_cfg1,
    "paged_fill_varlen": case_paged_fill_varlen,
    "varlen_causal": case_varlen_causal,
    "partial_rope": case_partial_rope,
    "gate_pack": case_gate_pack,
    "gdn_decode": case_gdn_decode,
    "gdn_sequential": case_gdn_sequential,
    "gdn_chunked": case_gdn_chunked,
    "glue_conv4": case_glue_conv4,
    "glue_norms": case_glue_norms,
    "glue_matmul": case_glue_matmul,
    "glue_gdn_decode_layer": case_glue_gdn_decode_layer,
    "glue_attn_decode_layer": case_glue_attn_decode_layer,
}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path to the reference checkout")
    ap.add_argument("--only", nargs="*", default=None)
    args = ap.parse_args()
    sys.path.insert(0, str(Path(args.reference).resolve()))
    pin = install_shims()
    print("pinned autotuners:", pin())
    for name, fn in CASES.items():
        if args.only and name not in args.only:
            continue
        t0 = time.time()
        data = fn()
        data = {k: (v.detach().clone().contiguous() if isinstance(v, torch.Tensor) else v)
                for k, v in data.items()}
        path = HERE / f"{name}.pt"
        torch.save(data, path)
        print(f"{name:24s} {time.time() - t0:7.1f}s  {path.stat().st_size / 1e6:6.2f} MB")


if __name__ == "__main__":
    main()
