"""CPU checks of the PyTorch glue operators that surround the CUDA path in whole-model stepping (b200attn/glue.py):
the packed depthwise conv against per-sequence convolution with zero history, the decode conv continuing a prefill,
and the packed conv-state extraction.  (The CUDA operators themselves have no CPU path.)"""
import sys
from pathlib import Path

import torch
import torch.nn.functional as F

sys.path.insert(0, str(Path(__file__).resolve().parents[1] / "qwen3_5-triton-inference-engine_b200"))


def _load_glue():
    import importlib.util
    path = Path(__file__).resolve().parents[1] / "qwen3_5-triton-inference-engine_b200" / "b200attn" / "glue.py"
    spec = importlib.util.spec_from_file_location("b200attn_glue_cpu", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _conv_one(x, w):
    total = x.shape[0]
    padded = F.pad(x.float(), (0, 0, 3, 0))
    return F.silu(sum(padded[r: r + total] * w.float()[:, r] for r in range(4))).to(x.dtype)


def test_packed_conv_matches_per_sequence():
    glue = _load_glue()
    gen = torch.Generator().manual_seed(0)
    lengths, chans = [1, 2, 3, 4, 9, 17], 48
    x = torch.randn(sum(lengths), chans, generator=gen).to(torch.bfloat16)
    w = (torch.randn(chans, 4, generator=gen) * 0.5).to(torch.bfloat16)
    starts = torch.cat([torch.full((n,), sum(lengths[:i]), dtype=torch.int32) for i, n in enumerate(lengths)])
    got = glue.depthwise_causal_conv4_prefill(x, w, starts)
    off = 0
    for n in lengths:
        assert torch.equal(got[off: off + n], _conv_one(x[off: off + n], w))
        off += n


def test_decode_conv_continues_prefill():
    glue = _load_glue()
    gen = torch.Generator().manual_seed(1)
    lengths, chans = [2, 5, 11], 32
    total = sum(lengths)
    x = torch.randn(total, chans, generator=gen).to(torch.bfloat16)
    nxt = torch.randn(len(lengths), chans, generator=gen).to(torch.bfloat16)
    w = (torch.randn(chans, 4, generator=gen) * 0.5).to(torch.bfloat16)
    cu = torch.tensor([0] + list(torch.tensor(lengths).cumsum(0)), dtype=torch.int32)
    state = torch.full((len(lengths), 4, chans), 7.0, dtype=torch.bfloat16)
    glue.conv_state_from_packed_prefill(state, x, cu)
    out = glue.depthwise_causal_conv4_decode(nxt, state, w.t().contiguous())
    off = 0
    for b, n in enumerate(lengths):
        full = _conv_one(torch.cat((x[off: off + n], nxt[b: b + 1])), w)
        assert torch.equal(out[b], full[-1])
        assert torch.equal(state[b, -1], nxt[b])
        off += n


def test_norms_and_gates_shapes():
    glue = _load_glue()
    gen = torch.Generator().manual_seed(2)
    x = torch.randn(3, 16, 128, generator=gen).to(torch.bfloat16)
    q_n, k_n, beta, g = glue.gdn_qk_norm_gates(x, x, torch.randn(3, 16, generator=gen), torch.randn(3, 16, generator=gen),
                                               torch.rand(16, generator=gen), torch.zeros(16))
    assert q_n.dtype == torch.bfloat16 and beta.dtype == torch.float32 and (g <= 0).all()
    assert torch.allclose(k_n.float().pow(2).sum(-1), torch.ones(3, 16), atol=2e-2)
    assert torch.allclose(q_n.float().pow(2).sum(-1), torch.full((3, 16), 1 / 128), atol=2e-4)
    y = glue.qwen_rmsnorm(x, torch.zeros(128, dtype=torch.bfloat16), 1e-6)
    assert torch.allclose(y.float().pow(2).mean(-1), torch.ones(3, 16), atol=2e-2)
    table = torch.eye(4, dtype=torch.bfloat16).repeat(2, 1)
    ids = glue.lm_head_argmax(torch.eye(4, dtype=torch.bfloat16), table, last_only=False)
    assert ids.tolist() == [0, 1, 2, 3]      # ties go to the lowest index
    assert int(glue.lm_head_argmax(torch.eye(4, dtype=torch.bfloat16), table)) == 3
