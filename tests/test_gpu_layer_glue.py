"""GPU parity of the single-launch row-wise layer operators (csrc/layer_glue.cu) against the eager PyTorch
restatements of the reference operators in b200attn/glue.py (same fp32 math and rounding points): at most one bf16
ulp apart (transcendentals come from different libraries), gates to 1e-6 relative."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def mods():
    from b200attn import glue, ops
    return ops, glue


def _ulp_close(a, b, ulps=1):
    a, b = a.float(), b.float()
    tol = ulps * 2.0 ** -8 * torch.maximum(a.abs(), b.abs()) + 1e-30
    assert bool(((a - b).abs() <= tol).all()), f"max diff {(a - b).abs().max().item()}"


def _prompt_close(a, b, what):
    """Prompt-sized forms (1024 rows and more): a million elements meet bf16 rounding boundaries that a different
    summation order or the fast exponential moves, so: never more than one bf16 ulp (2^-7 relative) apart, and at most
    1 % of the elements different at all."""
    assert a.shape == b.shape and a.dtype == b.dtype
    _ulp_close(a, b, ulps=2)
    differing = (a != b).float().mean().item()
    assert differing <= 0.01, f"{what}: {differing:.4f} of the elements differ"


@pytest.mark.parametrize("rows,dim", [(1, 1024), (32, 1024), (257, 256), (5, 2048)])
def test_add_rmsnorm(mods, rows, dim):
    ops, glue = mods
    gen = torch.Generator().manual_seed(rows * 7 + dim)
    x = torch.randn(rows, dim, generator=gen).to(torch.bfloat16).to(DEV)
    res = torch.randn(rows, dim, generator=gen).to(torch.bfloat16).to(DEV)
    w = (torch.randn(dim, generator=gen) * 0.1).to(torch.bfloat16).to(DEV)
    _ulp_close(ops.add_rmsnorm(x, w, 1e-6), glue.qwen_rmsnorm(x, w, 1e-6))
    total, norm = ops.add_rmsnorm(x, w, 1e-6, residual=res)
    ref_total = glue.residual_add(x, res)
    assert torch.equal(total, ref_total)
    _ulp_close(norm, glue.qwen_rmsnorm(ref_total, w, 1e-6))


@pytest.mark.parametrize("rows,dim", [(1027, 1024), (4096, 256), (1025, 2048), (1030, 512), (1024, 768)])
def test_add_rmsnorm_prompt_sized(mods, rows, dim):
    """From 1024 rows the operator runs its warp-per-row form (dims 256 / 512 / 1024 / 2048; 768 stays on the
    CTA-per-row form): the sum stays bit-exact, the norm within one bf16 ulp."""
    ops, glue = mods
    gen = torch.Generator().manual_seed(rows * 7 + dim)
    x = torch.randn(rows, dim, generator=gen).to(torch.bfloat16).to(DEV)
    res = torch.randn(rows, dim, generator=gen).to(torch.bfloat16).to(DEV)
    w = (torch.randn(dim, generator=gen) * 0.1).to(torch.bfloat16).to(DEV)
    _prompt_close(ops.add_rmsnorm(x, w, 1e-6), glue.qwen_rmsnorm(x, w, 1e-6), "norm")
    total, norm = ops.add_rmsnorm(x, w, 1e-6, residual=res)
    ref_total = glue.residual_add(x, res)
    assert torch.equal(total, ref_total)
    _prompt_close(norm, glue.qwen_rmsnorm(ref_total, w, 1e-6), "add + norm")
    fused = torch.randn(131, 5120, generator=gen).to(torch.bfloat16).to(DEV)   # head views: 1048 rows of 256
    w256 = (torch.randn(256, generator=gen) * 0.1).to(torch.bfloat16).to(DEV)
    view = fused[:, :2048].view(131, 8, 256)
    _prompt_close(ops.add_rmsnorm(view, w256, 1e-6), glue.qwen_rmsnorm(view, w256, 1e-6), "head views")


def test_rmsnorm_on_head_views(mods):
    """q / k norms read column views of the fused projection: [n, H, 256] with strides (5120, 256, 1)."""
    ops, glue = mods
    gen = torch.Generator().manual_seed(3)
    fused = torch.randn(9, 5120, generator=gen).to(torch.bfloat16).to(DEV)
    w = (torch.randn(256, generator=gen) * 0.1).to(torch.bfloat16).to(DEV)
    for view in (fused[:, :2048].view(9, 8, 256), fused[:, 4096:4608].view(9, 2, 256)):
        out = ops.add_rmsnorm(view, w, 1e-6)
        assert out.is_contiguous() and out.shape == view.shape
        _ulp_close(out, glue.qwen_rmsnorm(view, w, 1e-6))


@pytest.mark.parametrize("rows", [1, 32, 300])
def test_swiglu(mods, rows):
    ops, glue = mods
    gen = torch.Generator().manual_seed(rows)
    inter = 3584
    gu = (torch.randn(rows, 2 * inter, generator=gen) * 2).to(torch.bfloat16).to(DEV)
    _ulp_close(ops.swiglu_fused(gu, inter), glue.swiglu(gu[:, :inter], gu[:, inter:]))


@pytest.mark.parametrize("rows,inter", [(1027, 3584), (1024, 40), (2050, 1000)])
def test_swiglu_prompt_sized(mods, rows, inter):
    """From 1024 rows: the row-blocked form with the fast exponential, on the fused [rows, 2*inter] layout and on two
    separate column views."""
    ops, glue = mods
    from b200attn import glue_ops
    gen = torch.Generator().manual_seed(rows + inter)
    gu = (torch.randn(rows, 2 * inter, generator=gen) * 2).to(torch.bfloat16).to(DEV)
    gu[0, :8] = torch.tensor([-200.0, -90.0, -88.0, -30.0, 0.0, 30.0, 90.0, 200.0], dtype=torch.bfloat16)
    ref = glue.swiglu(gu[:, :inter], gu[:, inter:])
    _prompt_close(ops.swiglu_fused(gu, inter), ref, "fused layout")
    _prompt_close(glue_ops.swiglu(gu[:, :inter], gu[:, inter:]), ref, "column views")
    assert bool(torch.isfinite(ops.swiglu_fused(gu, inter).float()).all())


@pytest.mark.parametrize("lengths", [[1, 2, 3, 5, 64, 7, 1, 130], [4] * 9 + [3], [1] * 13, [258], [2, 1]])
@pytest.mark.parametrize("channels", [6144, 40])
def test_conv4_prefill_ragged(mods, lengths, channels):
    """A thread of the packed conv covers four consecutive tokens: sequences shorter than that window, sequence starts
    at every offset inside it and a token count that is not a multiple of four, against the eager restatement of the
    reference operator (one bf16 ulp: the kernel uses the fast exponential)."""
    _, glue = mods
    from b200attn import glue_ops
    gen = torch.Generator().manual_seed(sum(lengths) + channels)
    total = sum(lengths)
    x = torch.randn(total, channels, generator=gen).to(torch.bfloat16).to(DEV)
    w = (torch.randn(channels, 4, generator=gen) * 0.5).to(torch.bfloat16).to(DEV)
    starts = torch.tensor([s for s, n in zip(torch.tensor([0] + lengths[:-1]).cumsum(0).tolist(), lengths)
                           for _ in range(n)], dtype=torch.int32, device=DEV)
    ref = glue.depthwise_causal_conv4_prefill(x, w, starts)
    _prompt_close(glue_ops.depthwise_causal_conv4_prefill(x, w, starts), ref, "packed conv")
    _prompt_close(glue_ops.depthwise_causal_conv4_prefill(x, w.t().contiguous().t(), starts), ref, "[4,D] weight")
    if len(lengths) == 1:
        _prompt_close(glue_ops.depthwise_causal_conv4_prefill(x, w), ref, "no seq_start")


@pytest.mark.parametrize("tokens,heads", [(67, 16), (343, 3), (4096, 16)])
def test_gdn_row_operators_prompt_sized(mods, tokens, heads):
    """q/k norms + gates and the gated RMSNorm from 1024 (token, head) rows on: 16 lanes per row, eight rows per CTA,
    including a row count that leaves the last CTA partly empty (343 x 3 = 1029)."""
    ops, glue = mods
    from b200attn import glue_ops
    gen = torch.Generator().manual_seed(tokens + heads)
    kd = heads * 128
    fused = torch.randn(tokens, 4 * kd + 32, generator=gen).to(torch.bfloat16).to(DEV)   # rows stay 16-byte aligned
    a_log = (torch.rand(heads, generator=gen) * 2.7).to(DEV)
    dt_bias = (torch.randn(heads, generator=gen) * 0.5).to(torch.bfloat16).to(DEV)
    q, k = fused[:, :kd].view(tokens, heads, 128), fused[:, kd: 2 * kd].view(tokens, heads, 128)
    a, b = fused[:, 4 * kd: 4 * kd + heads], fused[:, 4 * kd + heads: 4 * kd + 2 * heads]
    rq, rk, rbeta, rg = glue.gdn_qk_norm_gates(q, k, a, b, a_log, dt_bias)
    q_n, k_n, beta, g = glue_ops.gdn_qk_norm_gates(q, k, a, b, a_log, dt_bias)
    _prompt_close(q_n, rq, "q_n")
    _prompt_close(k_n, rk, "k_n")
    assert torch.allclose(beta, rbeta, rtol=1e-5, atol=1e-7) and torch.allclose(g, rg, rtol=1e-5, atol=1e-7)
    x = torch.randn(tokens, heads, 128, generator=gen).to(torch.bfloat16).to(DEV)
    z = fused[:, 3 * kd: 4 * kd]
    w = (1 + 0.1 * torch.randn(128, generator=gen)).to(DEV)
    out = ops.gdn_gated_rmsnorm_fused(x, z, w)
    _prompt_close(out.view(tokens, heads, 128), glue.gdn_gated_rmsnorm(x, z.reshape(tokens, heads, 128), w), "gated norm")


@pytest.mark.parametrize("batch", [1, 32])
def test_gdn_decode_prep(mods, batch):
    ops, glue = mods
    gen = torch.Generator().manual_seed(50 + batch)
    heads, kd = 16, 2048
    fused = torch.randn(batch, 4 * kd + 2 * heads, generator=gen).to(torch.bfloat16).to(DEV)
    state = torch.randn(batch, 4, 3 * kd, generator=gen).to(torch.bfloat16).to(DEV)
    w4 = (torch.randn(4, 3 * kd, generator=gen) * 0.5).to(torch.bfloat16).to(DEV)
    a_log = (torch.rand(heads, generator=gen) * 2.7).to(DEV)
    dt_bias = (torch.randn(heads, generator=gen) * 0.5).to(torch.bfloat16).to(DEV)
    qkv, a, b = fused[:, : 3 * kd], fused[:, 4 * kd: 4 * kd + heads], fused[:, 4 * kd + heads:]
    ref_state = state.clone()
    conv = glue.depthwise_causal_conv4_decode(qkv, ref_state, w4)
    rq, rk, rbeta, rg = glue.gdn_qk_norm_gates(conv[:, :kd].view(batch, heads, 128), conv[:, kd: 2 * kd].view(batch, heads, 128),
                                               a, b, a_log, dt_bias)
    q_n, k_n, v, beta, g = ops.gdn_decode_prep(qkv, state, w4, a, b, a_log, dt_bias, heads)
    assert torch.equal(state, ref_state)
    _ulp_close(v, conv[:, 2 * kd:].view(batch, heads, 128))
    _ulp_close(q_n, rq, ulps=2)
    _ulp_close(k_n, rk, ulps=2)
    assert torch.allclose(beta, rbeta, rtol=1e-5, atol=1e-7) and torch.allclose(g, rg, rtol=1e-5, atol=1e-7)


def test_gdn_gated_rmsnorm(mods):
    ops, glue = mods
    gen = torch.Generator().manual_seed(8)
    n, heads = 33, 16
    x = torch.randn(n, heads, 128, generator=gen).to(torch.bfloat16).to(DEV)
    fused = torch.randn(n, 8224, generator=gen).to(torch.bfloat16).to(DEV)
    z = fused[:, 6144:8192]
    w = (1 + 0.1 * torch.randn(128, generator=gen)).to(DEV)
    out = ops.gdn_gated_rmsnorm_fused(x, z, w)
    _ulp_close(out.view(n, heads, 128), glue.gdn_gated_rmsnorm(x, z.reshape(n, heads, 128), w))


@pytest.mark.parametrize("prefetch", [0, 1 | 4])
@pytest.mark.parametrize("batch,form", [(1, 1), (32, 1), (1, 3), (32, 3), (40, 3)])
def test_gdn_decode_fused_equals_chain(mods, batch, form, prefetch):
    """One-launch Gated-DeltaNet decode mixer against prep -> recurrent_decode -> gated RMSNorm over three steps
    (conv state and recurrent state carried in place), in both of its forms: 1 = a head's state in registers, 3 = the
    state streamed through a ring of [128 x 32] boxes (40 sequences x 16 heads are more heads than CTAs fit the GPU,
    so some CTAs take a second head).  In form 1 the chain's recurrence sums in the fused kernel's order and the
    outputs agree to two bf16 ulps: the comparison is then about the fusion, not about fp32 summation order.  The ring
    mixer sums a column in four row groups, the ring recurrence of the chain in eight: an output that nearly cancels
    moves by more than two bf16 ulps of itself between orders, so there the output bar is two ulps of a value of
    order one plus a small absolute term; conv state (bit-exact) and recurrent state (1e-5) keep their bars."""
    from b200attn import _lib
    ops, glue = mods
    _lib.call("b200_gdn_recurrent_decode_form", form)
    try:
        _fused_against_chain(ops, batch, prefetch, same_order=form == 1)
    finally:
        _lib.call("b200_gdn_recurrent_decode_form", 0)


@pytest.mark.parametrize("batch,heads", [(48, 16), (256, 16), (100, 4), (37, 9)])
def test_gdn_decode_fused_forms_agree(mods, batch, heads):
    """The form the sizes choose (ring from more than two heads per SM on; at 256 sequences every CTA walks seven
    heads; head counts other than sixteen) against the register form on the same inputs: conv state bit-equal,
    recurrent state and output to summation-order accuracy."""
    from b200attn import _lib
    ops, _ = mods
    gen = torch.Generator().manual_seed(17)
    kd = heads * 128
    w4 = (torch.randn(4, 3 * kd, generator=gen) * 0.5).to(torch.bfloat16).to(DEV)
    a_log = (torch.rand(heads, generator=gen) * 2.7).to(DEV)
    dt_bias = (torch.randn(heads, generator=gen) * 0.5).to(torch.bfloat16).to(DEV)
    norm_w = (1 + 0.1 * torch.randn(128, generator=gen)).to(DEV)
    conv = torch.randn(batch, 4, 3 * kd, generator=gen).to(torch.bfloat16).to(DEV)
    state = (torch.randn(batch, heads, 128, 128, generator=gen) * 0.1).to(DEV)
    fused = torch.randn(batch, 4 * kd + 2 * heads, generator=gen).to(torch.bfloat16).to(DEV)
    results = []
    for form in (1, 0):
        _lib.call("b200_gdn_recurrent_decode_form", form)
        try:
            c, s = conv.clone(), state.clone()
            out = ops.gdn_decode_fused(fused, c, w4, a_log, dt_bias, norm_w, s, heads)
            results.append((c, s, out))
        finally:
            _lib.call("b200_gdn_recurrent_decode_form", 0)
    torch.cuda.synchronize()
    assert _lib.load().b200_wait_timed_out() == 0
    assert torch.equal(results[0][0], results[1][0])
    assert torch.allclose(results[0][1], results[1][1], rtol=1e-5, atol=1e-6)
    close = ((results[0][2].float() - results[1][2].float()).abs()
             <= 2.0 ** -6 * results[0][2].float().abs() + 2e-3)
    assert close.float().mean().item() > 0.999


def _fused_against_chain(ops, batch, prefetch, same_order=True):
    gen = torch.Generator().manual_seed(90 + batch)
    heads, kd = 16, 2048
    w4 = (torch.randn(4, 3 * kd, generator=gen) * 0.5).to(torch.bfloat16).to(DEV)
    a_log = (torch.rand(heads, generator=gen) * 2.7).to(DEV)
    dt_bias = (torch.randn(heads, generator=gen) * 0.5).to(torch.bfloat16).to(DEV)
    norm_w = (1 + 0.1 * torch.randn(128, generator=gen)).to(DEV)
    conv_a = torch.randn(batch, 4, 3 * kd, generator=gen).to(torch.bfloat16).to(DEV)
    state_a = (torch.randn(batch, heads, 128, 128, generator=gen) * 0.1).to(DEV)
    conv_b, state_b = conv_a.clone(), state_a.clone()
    for step in range(3):
        fused = torch.randn(batch, 4 * kd + 2 * heads, generator=gen).to(torch.bfloat16).to(DEV)
        q_n, k_n, v, beta, g = ops.gdn_decode_prep(fused[:, : 3 * kd], conv_a, w4, fused[:, 4 * kd: 4 * kd + heads],
                                                   fused[:, 4 * kd + heads:], a_log, dt_bias, heads)
        core = ops.gdn_recurrent_decode(q_n, k_n, v, beta, g, state_a)
        ref = ops.gdn_gated_rmsnorm_fused(core, fused[:, 3 * kd: 4 * kd], norm_w)
        out = ops.gdn_decode_fused(fused, conv_b, w4, a_log, dt_bias, norm_w, state_b, heads, overlap=prefetch)
        assert torch.equal(conv_a, conv_b)
        assert torch.allclose(state_a, state_b, rtol=1e-5, atol=1e-6)
        if same_order:
            _ulp_close(out, ref, ulps=2)
        else:
            assert torch.allclose(out.float(), ref.float(), rtol=2.0 ** -6, atol=4e-3)


@pytest.mark.parametrize("m,n,k", [(32, 8224, 1024), (1, 5120, 1024), (17, 7168, 1024), (32, 248320, 1024), (8, 512, 256),
                                   (32, 1024, 1280), (32, 1024, 2048), (32, 1024, 3584), (5, 256, 2048), (17, 40, 1536),
                                   (32, 4096, 7168), (1, 8, 16384), (32, 4096, 2048), (3, 2400, 4096)])
def test_skinny_gemm(mods, m, n, k):
    """Weight-streaming decode GEMM against an fp32 matmul of the same bf16 operands (exact products, fp32
    accumulation on both sides: only the summation order and the final bf16 rounding differ)."""
    ops, _ = mods
    gen = torch.Generator().manual_seed(m * 131 + n)
    x = torch.randn(m, k, generator=gen).to(torch.bfloat16).to(DEV)
    w = (torch.randn(n, k, generator=gen) * 0.05).to(torch.bfloat16).to(DEV)
    y = ops.skinny_gemm(x, w)
    ref = x.float() @ w.float().t()
    assert y.shape == (m, n)
    err = (y.float() - ref).abs().max().item()
    assert err <= 2.0 ** -8 * ref.abs().max().item() + 1e-6, err
    assert ops.skinny_gemm_supports(m, n, k)
    # a strided input row view (a slice of a wider activation) gives the same result
    wide = torch.zeros(m, k + 64, dtype=torch.bfloat16, device=DEV)
    wide[:, :k] = x
    assert torch.equal(ops.skinny_gemm(wide[:, :k], w), y)


def test_overlapped_chain_in_graph_equals_plain(mods):
    """add_rmsnorm -> skinny_gemm -> gdn_decode_fused launched with every overlap flag (programmatic dependent launch:
    each kernel starts while its predecessor runs, the mixer pre-loads its states) and replayed from a CUDA graph with
    a NEW input every replay, against the same chain in plain stream order.  A kernel that read its predecessor's
    output before it was complete would see the previous replay's values."""
    ops, _ = mods
    gen = torch.Generator().manual_seed(7)
    batch, heads, kd, hidden = 4, 16, 2048, 256
    w_in = (torch.randn(4 * kd + 2 * heads, hidden, generator=gen) * 0.05).to(torch.bfloat16).to(DEV)
    w4 = (torch.randn(4, 3 * kd, generator=gen) * 0.5).to(torch.bfloat16).to(DEV)
    a_log = (torch.rand(heads, generator=gen) * 2.7).to(DEV)
    dt_bias = (torch.randn(heads, generator=gen) * 0.5).to(torch.bfloat16).to(DEV)
    norm_w = (1 + 0.1 * torch.randn(128, generator=gen)).to(DEV)
    ln = (torch.randn(hidden, generator=gen) * 0.1).to(torch.bfloat16).to(DEV)
    xs = [torch.randn(batch, hidden, generator=gen).to(torch.bfloat16).to(DEV) for _ in range(5)]
    conv0 = torch.randn(batch, 4, 3 * kd, generator=gen).to(torch.bfloat16).to(DEV)
    state0 = (torch.randn(batch, heads, 128, 128, generator=gen) * 0.1).to(DEV)

    def run(overlapped: bool):
        conv, state, x = conv0.clone(), state0.clone(), xs[0].clone()
        out = torch.zeros(batch, kd, dtype=torch.bfloat16, device=DEV)
        chain = ops.OVERLAP_START | ops.OVERLAP_TRIGGER if overlapped else 0
        last = ops.OVERLAP_START | ops.OVERLAP_PREFETCH if overlapped else 0

        def step():
            h = ops.add_rmsnorm(x, ln, 1e-6, overlap=chain)
            fused = ops.skinny_gemm(h, w_in, overlap=chain)
            out.copy_(ops.gdn_decode_fused(fused, conv, w4, a_log, dt_bias, norm_w, state, heads, overlap=last))

        step()
        outs = [out.clone()]
        graph = None
        if overlapped:
            graph = torch.cuda.CUDAGraph()
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side), torch.cuda.graph(graph, stream=side):
                step()
            torch.cuda.current_stream().wait_stream(side)
        for nxt in xs[1:]:
            x.copy_(nxt)
            graph.replay() if graph is not None else step()
            outs.append(out.clone())
        torch.cuda.synchronize()
        return outs, state, conv

    plain, fast = run(False), run(True)
    for a, b in zip(plain[0], fast[0]):
        assert torch.equal(a, b)
    assert torch.equal(plain[1], fast[1]) and torch.equal(plain[2], fast[2])


@pytest.mark.parametrize("m,k,inter", [(32, 1024, 3584), (4, 256, 512), (17, 1280, 1000), (1, 128, 8), (32, 1024, 40)])
def test_skinny_gemm_swiglu_equals_chain(mods, m, k, inter):
    """Gate/up projection with the SwiGLU in its epilogue against skinny_gemm -> swiglu: the same products in the same
    order, the same rounding of the projection to bf16 in between, so the same bytes.  `inter` values that are not a
    multiple of the 32 outputs a CTA covers exercise the tiles that hang over the end of the gate (and up) rows."""
    ops, _ = mods
    gen = torch.Generator().manual_seed(m + k + inter)
    x = torch.randn(m, k, generator=gen).to(torch.bfloat16).to(DEV)
    w = (torch.randn(2 * inter, k, generator=gen) * 0.05).to(torch.bfloat16).to(DEV)
    ref = ops.swiglu_fused(ops.skinny_gemm(x, w), inter)
    y = ops.skinny_gemm(x, w, swiglu=True)
    assert y.shape == ref.shape == (m, inter)
    assert torch.equal(y, ref)


@pytest.mark.parametrize("rows,n", [(32, 248320), (1, 8), (5, 1000), (1024, 64), (3, 40004)])
def test_argmax_rows_equals_torch(mods, rows, n):
    """Row arg-max of fp32 logits against torch.argmax (first maximal value wins): random rows, rows whose maximum
    occurs several times (in different slices and inside one 16-byte load), a constant row, a row of -inf, a row view
    with a larger stride; the workspace must be all zero again after every call."""
    ops, _ = mods
    gen = torch.Generator().manual_seed(rows + n)
    wide = torch.randn(rows, n + 8, generator=gen)
    logits = wide[:, :n]                               # row stride n + 8
    top = logits.max(dim=1).values
    for r in range(0, rows, 3):                        # plant duplicates of the maximum
        for c in torch.randint(0, n, (4,), generator=gen).tolist():
            logits[r, c] = top[r]
        c0 = int(torch.randint(0, n - 1, (1,), generator=gen))
        logits[r, c0] = logits[r, c0 + 1] = top[r]
    if rows >= 3:
        logits[1] = 0.25
        logits[2] = float("-inf")
    dev_logits = wide.to(DEV)[:, :n]
    ws = ops.argmax_workspace(DEV)
    for _ in range(2):
        ids = ops.argmax_rows(dev_logits, ws)
        assert torch.equal(ids.cpu(), torch.argmax(logits, dim=1))
        assert int(ws.abs().sum()) == 0


@pytest.mark.parametrize("m,v,k", [(32, 248320, 1024), (5, 2048, 256), (1, 40, 128), (17, 100000, 1280)])
def test_lm_head_argmax(mods, m, v, k):
    """LM head + greedy sampling in one launch against the fp32 logits of the same bf16 operands: the chosen id's
    logit is the row maximum up to the fp32 summation order; with duplicated table rows (identical logits, computed
    by identical arithmetic) the lowest id wins; the workspace is zero again afterwards."""
    ops, _ = mods
    gen = torch.Generator().manual_seed(m + v + k)
    h = torch.randn(m, k, generator=gen).to(torch.bfloat16).to(DEV)
    table = (torch.randn(v, k, generator=gen) * 0.05).to(torch.bfloat16).to(DEV)
    ws = ops.argmax_workspace(DEV)
    ids = ops.lm_head_argmax(h, table, ws)
    logits = h.float() @ table.float().t()
    top = logits.max(dim=1).values
    picked = logits.gather(1, ids.view(-1, 1)).squeeze(1)
    assert ids.dtype == torch.int64 and int(ids.min()) >= 0 and int(ids.max()) < v
    assert torch.all(picked >= top - 1e-4 * top.abs().clamp_min(1.0)), (picked - top).min().item()
    assert int(ws.abs().sum()) == 0
    # ties: copy every row's winner to a few other rows, below and above it
    table2 = table.clone()
    expect = []
    for r in range(m):
        w = int(ids[r])
        twins = sorted({w, (w * 7 + 3) % v, (w + v // 2) % v})
        for tw in twins:
            table2[tw] = table[w]
        expect.append(twins)
    ids2 = ops.lm_head_argmax(h, table2, ws)
    logits2 = h.float() @ table2.float().t()
    for r in range(m):
        best = int(ids2[r])
        # a copied row of another sequence's winner may beat this row's old maximum: accept any exact-tie set
        ties = (logits2[r] >= logits2[r, best] - 1e-4 * max(1.0, abs(float(logits2[r, best])))).nonzero().flatten().tolist()
        assert best in ties
        same = [t for t in expect[r] if t in ties]
        if best in expect[r]:
            assert best == min(same)
    assert int(ws.abs().sum()) == 0
