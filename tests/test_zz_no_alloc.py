"""The allocation-free fused decode entry point against the regular one, through the C ABI.

`b200_fused_decode_attention_static` exists for hosts that may not allocate device memory (a serving runtime
that owns the whole GPU, a plugin inside another process, code under stream capture): its workspace is a fixed
array inside the library instead of a caller buffer.  It must give the same result as the regular entry point,
call after call, with whatever the previous call left in the shared array.  This file is named to be collected
last, so a failure here cannot hide the other tests behind `-x`; it also passes when run alone in a fresh process.
"""
import pytest
import torch

from helpers import bf16_randn, make_paged_case, maxabs, rope_inv_freq

pytestmark = pytest.mark.gpu
DEV = "cuda"
TOL = 2e-2  # same bar as the other decode-attention tests (bf16 output, max-abs)


def call_static(lib_call, t, kc, vc, inv, out):
    """Straight ctypes call of the C entry point: raw pointers, element strides, stream handle."""
    q, k_new, v_new, gate, bt, pos = t["q"], t["k_new"], t["v_new"], t["gate"], t["block_table"], t["pos"]
    batch, hq, d = q.shape
    lib_call("b200_fused_decode_attention_static", q.data_ptr(), q.stride(0), q.stride(1), k_new.data_ptr(),
             k_new.stride(0), k_new.stride(1), v_new.data_ptr(), v_new.stride(0), v_new.stride(1), gate.data_ptr(),
             gate.stride(0), kc.data_ptr(), vc.data_ptr(), kc.stride(0), kc.stride(1), kc.stride(2), vc.stride(0),
             vc.stride(1), vc.stride(2), kc.shape[0], bt.data_ptr(), bt.stride(0), pos.data_ptr(), inv.data_ptr(), 64,
             out.data_ptr(), batch, hq, k_new.shape[1], d, torch.cuda.current_stream().cuda_stream)


def test_static_workspace_matches_regular_entry_point_twice():
    from b200attn import _lib, ops

    lengths = [700, 33, 2049, 16, 0, 4000, 255, 1200]   # several sequences are cut across CTAs -> the workspace is used
    c = make_paged_case(lengths, seed=5, slack_tokens=4)
    t = {k: (v.to(DEV) if isinstance(v, torch.Tensor) else v) for k, v in c.items()}
    inv = rope_inv_freq().to(DEV)
    ws = ops.fused_decode_workspace(DEV)
    gen = torch.Generator().manual_seed(99)
    kc_a, vc_a = t["k_cache"].clone(), t["v_cache"].clone()   # regular entry point
    kc_b, vc_b = t["k_cache"].clone(), t["v_cache"].clone()   # allocation-free entry point
    for step in range(2):
        if step == 1:  # second call: next token of every sequence, fresh projections, same shared array
            t["pos"] = t["pos"] + 1
            t["q"] = bf16_randn(len(lengths), 8, 256, gen=gen).to(DEV)
            t["k_new"] = bf16_randn(len(lengths), 2, 256, gen=gen).to(DEV)
            t["v_new"] = bf16_randn(len(lengths), 2, 256, gen=gen).to(DEV)
        ref = ops.fused_decode_attention(t["q"], t["k_new"], t["v_new"], t["gate"], kc_a, vc_a, t["block_table"],
                                         t["pos"], inv, 64, ws)
        out = torch.empty_like(ref)
        before = torch.cuda.memory_allocated()
        call_static(_lib.call, t, kc_b, vc_b, inv, out)
        assert torch.cuda.memory_allocated() == before
        torch.cuda.synchronize()
        assert maxabs(out, ref) <= TOL, f"call {step}"
        assert torch.equal(kc_a, kc_b) and torch.equal(vc_a, vc_b), f"cache contents differ after call {step}"
    assert _lib.load().b200_wait_timed_out() == 0


def test_static_workspace_rejects_oversized_batch():
    from b200attn import _lib

    z = torch.zeros(1, device=DEV)
    with pytest.raises(_lib.B200Error, match="built-in workspace"):
        _lib.call("b200_fused_decode_attention_static", z.data_ptr(), 2048, 256, z.data_ptr(), 512, 256, z.data_ptr(),
                  512, 256, z.data_ptr(), 2048, z.data_ptr(), z.data_ptr(), 8192, 4096, 256, 8192, 4096, 256, 4,
                  z.data_ptr(), 8, z.data_ptr(), z.data_ptr(), 64, z.data_ptr(), 513, 8, 2, 256, None)
