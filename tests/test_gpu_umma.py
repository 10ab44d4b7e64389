"""tcgen05 / TMEM / tensor-map TMA building blocks against torch.matmul (bf16 inputs, fp32 accumulate)."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("mode", [0, 1, 2])
def test_umma_selftest(mode):
    from b200attn import _lib

    gen = torch.Generator().manual_seed(10 + mode)
    if mode == 0:
        a = torch.randn(128, 256, generator=gen).to(torch.bfloat16)
        b = torch.randn(64, 256, generator=gen).to(torch.bfloat16)
        ref = a.float() @ b.float().t()
    else:
        a = torch.randn(128, 64, generator=gen).to(torch.bfloat16)
        b = torch.randn(64, 256, generator=gen).to(torch.bfloat16)
        ref = a.float() @ b.float()
    ad, bd = a.to(DEV), b.to(DEV)
    c = torch.full(ref.shape, float("nan"), device=DEV)
    _lib.call("b200_selftest_umma", mode, ad.data_ptr(), bd.data_ptr(), c.data_ptr(), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert _lib.load().b200_wait_timed_out() == 0
    err = (c.cpu() - ref).abs().max().item()
    assert err < 1e-3 * max(1.0, ref.abs().max().item()), f"mode {mode}: max abs err {err}"
