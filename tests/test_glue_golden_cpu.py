"""The PyTorch restatements of the operators around the path (b200attn/glue.py) against outputs of the REFERENCE's own
kernels (tests/golden/glue_*.pt, made by tests/golden/make_golden.py under the Triton interpreter).  glue.py is what a
shape outside a CUDA kernel's rules falls back to on the GPU, and the CPU-checkable statement of the same arithmetic."""
import importlib.util
from pathlib import Path

import torch

from helpers import assert_bf16_close

PKG = Path(__file__).resolve().parents[1] / "qwen3_5-triton-inference-engine_b200"


def _glue():
    spec = importlib.util.spec_from_file_location("b200attn_glue_cpu2", PKG / "b200attn" / "glue.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_conv4_against_reference(golden):
    glue, g = _glue(), golden("glue_conv4")
    assert_bf16_close(glue.depthwise_causal_conv4_prefill(g["x"], g["weight"], g["seq_start"]), g["prefill_packed"],
                      what="packed conv", max_mismatch_frac=0.01)
    assert_bf16_close(glue.depthwise_causal_conv4_prefill(g["x"][:3], g["weight"]), g["prefill_single"],
                      what="single conv", max_mismatch_frac=0.01)
    state = g["state_garbage"].clone()
    glue.conv_state_from_packed_prefill(state, g["x"], g["cu_seqlens"])
    assert torch.equal(state, g["state_from_packed"])          # byte-equal, as the reference's own test demands
    st = g["decode_state_in"].clone()
    out = glue.depthwise_causal_conv4_decode(g["decode_fused_row"][:, :6144], st, g["weight4"])
    assert torch.equal(st, g["decode_state_out"])
    assert_bf16_close(out, g["decode_out"], what="decode conv", max_mismatch_frac=0.01)


def test_norms_and_gates_against_reference(golden):
    glue, g = _glue(), golden("glue_norms")
    assert_bf16_close(glue.qwen_rmsnorm(g["rms.x2"], g["rms.w1024"], 1e-6), g["rms.out2"], what="rmsnorm rows",
                      max_mismatch_frac=0.01)
    view = g["rms.fused"][:, :2048].view(3, 8, 256)
    assert_bf16_close(glue.qwen_rmsnorm(view, g["rms.w256"], 1e-6), g["rms.out3"], what="rmsnorm heads",
                      max_mismatch_frac=0.01)
    t, h, d = 5, 16, 128
    conv, ab = g["qk.conv"], g["qk.ab"]
    q_n, k_n, beta, gg = glue.gdn_qk_norm_gates(conv[:, : h * d].view(t, h, d), conv[:, h * d: 2 * h * d].view(t, h, d),
                                                ab[:, :h], ab[:, h:], g["qk.a_log"], g["qk.dt_bias"])
    assert_bf16_close(q_n, g["qk.q_n"], what="q_n", max_mismatch_frac=0.01)
    assert_bf16_close(k_n, g["qk.k_n"], what="k_n", max_mismatch_frac=0.01)
    torch.testing.assert_close(beta, g["qk.beta"], rtol=2e-6, atol=1e-7)
    torch.testing.assert_close(gg, g["qk.g"], rtol=5e-6, atol=1e-7)
    z = g["gn.z_rows"][:, : h * d].view(t, h, d)
    assert_bf16_close(glue.gdn_gated_rmsnorm(g["gn.x"], z, g["gn.weight"]), g["gn.out"], what="gated norm",
                      max_mismatch_frac=0.01)
    gu = g["swiglu.gate_up"]
    assert_bf16_close(glue.swiglu(gu[:, :3584], gu[:, 3584:]), g["swiglu.out"], what="swiglu", max_mismatch_frac=0.01)
    assert torch.equal(glue.embedding_gather(g["gather.ids"], g["gather.table"]), g["gather.out"])


def test_matmul_and_argmax_against_reference(golden):
    glue, g = _glue(), golden("glue_matmul")
    for m in (1, 5):
        assert_bf16_close(glue.gemm_2d(g[f"gemm.x{m}"], g["gemm.w"]), g[f"gemm.y{m}"], what=f"gemm M={m}",
                          max_mismatch_frac=0.05)
    assert torch.equal(glue.lm_head_argmax(g["argmax.rows"], g["argmax.table"], last_only=False), g["argmax.ids"])
    assert int(glue.lm_head_argmax(g["argmax.rows"], g["argmax.table"], last_only=True)) == int(g["argmax.last"])
