"""GPU parity of the paged KV writers and the paged decode attention (drop-in chain and fused kernel).

Every call goes through the `wy_lib::*` operators / Python boundary into the C ABI of libb200attn.so.
Bars: page/index work bit-exact; bf16 attention outputs within max-abs 2e-2 of the fp32 oracle.
"""
import pytest
import torch

from helpers import bf16_randn, cdiv, make_paged_case, maxabs, rope_inv_freq
from oracle import reference_ops as O

pytestmark = pytest.mark.gpu
DEV = "cuda"
TOL = 2e-2  # max-abs on bf16 attention outputs vs the fp32 oracle


@pytest.fixture(scope="module")
def ops():
    from b200attn import ops as _ops
    return _ops


def to_dev(d):
    return {k: (v.to(DEV) if isinstance(v, torch.Tensor) else v) for k, v in d.items()}


def no_timeouts():
    import b200attn
    assert b200attn.load().b200_wait_timed_out() == 0, "a kernel gave up waiting for a staged copy"


# --------------------------------------------------------------------------- KV writers (bit-exact)
def test_append_and_chain_cfg1_golden(ops, golden, monkeypatch):
    """The runner's decode symbol against the reference's own outputs on config 1: in its three-launch form the scratch
    tensors must hold the reference's partials; in its one-launch form only the result and the caches are compared."""
    monkeypatch.setattr(ops, "DECODE_CALL_ONE_LAUNCH", False)
    g = golden("paged_decode_cfg1")
    d = to_dev(g)
    kc, vc = d["k_cache_in"].clone(), d["v_cache_in"].clone()
    b, hq, dim = g["q"].shape
    m = torch.full((b, hq, 128), 7.0, device=DEV)
    l = torch.full((b, hq, 128), 3.0, device=DEV)
    acc = torch.full((b, hq, 128, dim), -5.0, device=DEV)
    out = ops.call_paged_gqa_attention_decode_triton(d["q"], d["k_new"], d["v_new"], kc, vc, d["block_table"], d["pos"],
                                                     (m, l, acc))
    torch.cuda.synchronize()
    no_timeouts()
    assert torch.equal(kc.cpu(), g["k_cache_out"]) and torch.equal(vc.cpu(), g["v_cache_out"])
    keep = int(g["partial_keep"])
    mc, lc, ac = m.cpu(), l.cpu(), acc.cpu()
    assert torch.equal(torch.isinf(mc[:, :, :keep]), torch.isinf(g["m_partial_head"]))
    fin = ~torch.isinf(g["m_partial_head"])
    assert maxabs(mc[:, :, :keep][fin], g["m_partial_head"][fin]) < 1e-4
    assert maxabs(lc[:, :, :keep], g["l_partial_head"]) < 1e-3
    assert maxabs(ac[:, :, :keep], g["acc_partial_head"]) < 5e-2  # p is rounded to bf16: one flip moves acc by ~|v|*2^-9
    assert torch.isinf(mc[:, :, keep:]).all() and (lc[:, :, keep:] == 0).all() and (ac[:, :, keep:] == 0).all()
    assert maxabs(out, g["out"]) <= 2 ** -7
    exact = O.paged_decode_exact(g["q"], g["k_cache_out"], g["v_cache_out"], g["block_table"], (g["pos"] + 1).tolist())
    assert maxabs(out, exact) < TOL
    monkeypatch.setattr(ops, "DECODE_CALL_ONE_LAUNCH", True)
    kc1, vc1 = d["k_cache_in"].clone(), d["v_cache_in"].clone()
    out1 = ops.call_paged_gqa_attention_decode_triton(d["q"], d["k_new"], d["v_new"], kc1, vc1, d["block_table"], d["pos"],
                                                      (m, l, acc))
    torch.cuda.synchronize()
    no_timeouts()
    assert torch.equal(kc1.cpu(), g["k_cache_out"]) and torch.equal(vc1.cpu(), g["v_cache_out"])
    assert maxabs(out1, g["out"]) <= 2 ** -7 and maxabs(out1, exact) < TOL
    assert torch.equal(m.cpu(), mc) and torch.equal(acc.cpu(), ac)   # the one-launch form leaves the scratch alone


@pytest.mark.parametrize("lengths", [[16], [17], [1], [16, 16], [7, 100, 1, 64], [128] * 8, [1, 1, 1, 1000]])
@pytest.mark.parametrize("shuffle", [False, True])
def test_fill_varlen_bit_exact(ops, lengths, shuffle):
    """The reference's own self-test grid (gqa_attention_decode_paged.py:1092-1102): byte equality, non-zero
    initial pool, unallocated pages untouched, shuffled page table."""
    gen = torch.Generator().manual_seed(sum(lengths) + 7 * len(lengths) + int(shuffle))
    batch, total, hkv, d = len(lengths), sum(lengths), 2, 256
    pps = cdiv(max(lengths), 16)
    num_pages = batch * pps + 8
    order = torch.randperm(num_pages, generator=gen) if shuffle else torch.arange(num_pages)
    bt = order[: batch * pps].view(batch, pps).to(torch.int32).contiguous()
    cu = torch.tensor([0] + list(torch.tensor(lengths).cumsum(0)), dtype=torch.int32)
    k_thd, v_thd = bf16_randn(total, hkv, d, gen=gen), bf16_randn(total, hkv, d, gen=gen)
    init_k, init_v = bf16_randn(num_pages, hkv, 16, d, gen=gen), bf16_randn(num_pages, hkv, 16, d, gen=gen)
    kr, vr = init_k.clone(), init_v.clone()
    O.paged_kv_fill_varlen(kr, vr, k_thd.permute(1, 0, 2), v_thd.permute(1, 0, 2), bt, cu)
    kc, vc = init_k.to(DEV), init_v.to(DEV)
    ops.paged_kv_fill_varlen(kc, vc, k_thd.to(DEV).permute(1, 0, 2), v_thd.to(DEV).permute(1, 0, 2), bt.to(DEV),
                             cu.to(DEV), max(lengths))
    assert torch.equal(kc.cpu(), kr) and torch.equal(vc.cpu(), vr)
    rest = order[batch * pps:]
    assert torch.equal(kc.cpu()[rest], init_k[rest])


def test_fill_varlen_golden(ops, golden):
    g = golden("paged_fill_varlen")
    for tag in ("a", "b"):
        kc, vc = g[f"{tag}.k_cache_in"].to(DEV), g[f"{tag}.v_cache_in"].to(DEV)
        ops.paged_kv_fill_varlen(kc, vc, g[f"{tag}.k_thd"].to(DEV).permute(1, 0, 2),
                                 g[f"{tag}.v_thd"].to(DEV).permute(1, 0, 2), g[f"{tag}.block_table"].to(DEV),
                                 g[f"{tag}.cu_seqlens"].to(DEV), int(g[f"{tag}.lengths"].max()))
        assert torch.equal(kc.cpu(), g[f"{tag}.k_cache_out"]) and torch.equal(vc.cpu(), g[f"{tag}.v_cache_out"])


def test_paged_kv_fill_single_sequence(ops):
    c = make_paged_case([40], seed=3)
    gen = torch.Generator().manual_seed(5)
    k, v = bf16_randn(2, 40, 256, gen=gen), bf16_randn(2, 40, 256, gen=gen)
    kr, vr = c["k_cache"].clone(), c["v_cache"].clone()
    O.paged_kv_fill_varlen(kr, vr, k, v, c["block_table"], torch.tensor([0, 40], dtype=torch.int32))
    kc, vc = c["k_cache"].to(DEV), c["v_cache"].to(DEV)
    ops.paged_kv_fill(kc, vc, k.to(DEV), v.to(DEV), c["block_table"][0].to(DEV))
    assert torch.equal(kc.cpu(), kr) and torch.equal(vc.cpu(), vr)


def test_append_strided_inputs_bit_exact(ops):
    """k_new / v_new arrive as slices of one fused projection row (engine/runner.py:469-471)."""
    c = make_paged_case([5, 31, 32, 700], seed=4)
    gen = torch.Generator().manual_seed(9)
    fused = bf16_randn(4, 5120, gen=gen)
    k_new = fused[:, 4096:4608].view(4, 2, 256)
    v_new = fused[:, 4608:].view(4, 2, 256)
    kr, vr = c["k_cache"].clone(), c["v_cache"].clone()
    O.paged_kv_append(kr, vr, k_new, v_new, c["block_table"], c["pos"])
    fd = fused.to(DEV)
    kc, vc = c["k_cache"].to(DEV), c["v_cache"].to(DEV)
    ops.paged_kv_append(kc, vc, fd[:, 4096:4608].view(4, 2, 256), fd[:, 4608:].view(4, 2, 256),
                        c["block_table"].to(DEV), c["pos"].to(DEV))
    assert torch.equal(kc.cpu(), kr) and torch.equal(vc.cpu(), vr)


# --------------------------------------------------------------------------- drop-in split / combine
@pytest.mark.parametrize("one_launch", [False, True])
@pytest.mark.parametrize("lengths", [[0], [15], [16], [1, 17, 255, 256, 2047, 2048], [4095, 33, 2100, 512], [6000]])
def test_decode_chain_vs_oracle(ops, lengths, one_launch, monkeypatch):
    """`call_paged_gqa_attention_decode_triton` in both of its forms: the reference's three launches through the scratch
    tensors (whose contents are then the reference's partial layout) and the single launch of the fused kernel without
    RoPE and gate (which leaves the scratch alone)."""
    monkeypatch.setattr(ops, "DECODE_CALL_ONE_LAUNCH", one_launch)
    c = make_paged_case(lengths, seed=100 + len(lengths) + lengths[0])
    d = to_dev(c)
    kc, vc = d["k_cache"].clone(), d["v_cache"].clone()
    scratch = tuple(torch.full_like(t, 3.0) for t in ops.allocate_split_scratch(8, 256, batch=len(lengths), device=DEV))
    out = ops.call_paged_gqa_attention_decode_triton(d["q"], d["k_new"], d["v_new"], kc, vc, d["block_table"], d["pos"],
                                                     scratch)
    torch.cuda.synchronize()
    no_timeouts()
    kr, vr = c["k_cache"].clone(), c["v_cache"].clone()
    O.paged_kv_append(kr, vr, c["k_new"], c["v_new"], c["block_table"], c["pos"])
    assert torch.equal(kc.cpu(), kr) and torch.equal(vc.cpu(), vr)
    exact = O.paged_decode_exact(c["q"], kr, vr, c["block_table"], (c["pos"] + 1).tolist())
    assert maxabs(out, exact) < TOL
    m, l, acc = (t.cpu() for t in scratch)
    if one_launch and len(lengths) >= 4:   # one or two sequences always take the three launches
        assert bool((m == 3.0).all() and (l == 3.0).all() and (acc == 3.0).all())
        return
    # inactive splits hold (-inf, 0, 0), like the reference kernel leaves them
    for b, n in enumerate(lengths):
        _, _, _, active = O.split_geometry(n)
        assert torch.isinf(m[b, :, active:]).all() and (l[b, :, active:] == 0).all() and (acc[b, :, active:] == 0).all()
        assert torch.isfinite(m[b, :, :active]).all()


def test_decode_chain_small_matches_rounding_model(ops):
    """Small case against the page-by-page oracle that rounds p to bf16 like the kernels do."""
    c = make_paged_case([37, 64, 100, 128, 3], seed=21)
    d = to_dev(c)
    kc, vc = d["k_cache"].clone(), d["v_cache"].clone()
    out = ops.call_paged_gqa_attention_decode_triton(d["q"], d["k_new"], d["v_new"], kc, vc, d["block_table"], d["pos"])
    kr, vr = c["k_cache"].clone(), c["v_cache"].clone()
    ref = O.paged_decode(c["q"], c["k_new"], c["v_new"], kr, vr, c["block_table"], c["pos"])
    assert maxabs(out, ref) <= 2 ** -6
    assert (out.float().cpu() - ref.float()).abs().mean().item() < 2e-4


def test_nan_in_unowned_slots_is_ignored(ops):
    """Slots past the context in the last page, and pages the sequence does not own, may hold NaN."""
    c = make_paged_case([21, 40], seed=8)
    nan = torch.tensor(float("nan"), dtype=torch.bfloat16)
    for b, n in enumerate(c["pos"].tolist()):
        page = int(c["block_table"][b, n // 16])
        c["k_cache"][page, :, n % 16 + 1:, :] = nan   # after the slot the appended token will take
        c["v_cache"][page, :, n % 16 + 1:, :] = nan
    c["k_cache"][c["unowned"]] = nan
    c["v_cache"][c["unowned"]] = nan
    d = to_dev(c)
    out = ops.call_paged_gqa_attention_decode_triton(d["q"], d["k_new"], d["v_new"], d["k_cache"], d["v_cache"],
                                                     d["block_table"], d["pos"])
    assert torch.isfinite(out.float()).all()
    ws = ops.fused_decode_workspace(DEV)
    d2 = to_dev(c)
    out2 = ops.fused_decode_attention(d2["q"], d2["k_new"], d2["v_new"], d2["gate"], d2["k_cache"], d2["v_cache"],
                                      d2["block_table"], d2["pos"], rope_inv_freq().to(DEV), 64, ws)
    assert torch.isfinite(out2.float()).all()


# --------------------------------------------------------------------------- fused decode kernel
@pytest.mark.parametrize("lengths", [[0], [1], [16], [37, 64, 100, 128], [0, 15, 16, 17, 31, 32, 33, 1000],
                                     [4096, 512, 33, 2049, 777, 1, 3000, 16], [32768], [600] * 64])
@pytest.mark.parametrize("partition", [0, 1, 2, 3])
def test_fused_decode_vs_oracle(ops, lengths, partition):
    """partition pins how the kernel cuts the KV pages over its CTAs (1 = equal page ranges with cross-CTA merges,
    2 = one whole segment per CTA, 3 = one segment per thread-block cluster, 0 = the kernel's own choice), so that every
    form is checked on every length set it can take."""
    if partition == 2 and 2 * len(lengths) > torch.cuda.get_device_properties(0).multi_processor_count:
        pytest.skip("whole segments need no more segments than SMs")
    if partition == 3 and 2 * len(lengths) > 64:
        pytest.skip("a cluster per segment needs at most 64 segments")
    c = make_paged_case(lengths, seed=300 + len(lengths) + lengths[0])
    inv = rope_inv_freq()
    d = to_dev(c)
    ws = ops.fused_decode_workspace(DEV)
    kc, vc = d["k_cache"].clone(), d["v_cache"].clone()
    out = ops.fused_decode_attention(d["q"], d["k_new"], d["v_new"], d["gate"], kc, vc, d["block_table"], d["pos"],
                                     inv.to(DEV), 64, ws, partition=partition)
    torch.cuda.synchronize()
    no_timeouts()
    assert int(ws[:8192].view(torch.int32).abs().sum()) == 0, "segment counters must return to zero"
    kr, vr = c["k_cache"].clone(), c["v_cache"].clone()
    big = max(lengths) > 300 or len(lengths) > 8
    ref = O.fused_decode_attention(c["q"], c["k_new"], c["v_new"], c["gate"], kr, vr, c["block_table"], c["pos"], inv,
                                   64, exact=big)
    assert torch.equal(vc.cpu(), vr)                       # V rows are copies: bit-exact
    assert maxabs(kc, kr) <= 2 ** -6                       # K rows went through sin/cos: one bf16 ulp at |x| < 4
    assert (kc.cpu() != kr).float().mean().item() < 1e-3
    assert maxabs(out, ref) < TOL
    # same call again on the updated cache and the same workspace: stale partials must not leak
    out2 = ops.fused_decode_attention(d["q"], d["k_new"], d["v_new"], d["gate"], kc, vc, d["block_table"], d["pos"],
                                      inv.to(DEV), 64, ws, partition=partition)
    assert torch.equal(out2, out)


def test_fused_matches_dropin_chain(ops):
    """Fused kernel == partial_rope x2 -> append -> split -> combine -> gate_pack built from the drop-in operators."""
    lengths = [5, 250, 1024, 77]
    c = make_paged_case(lengths, seed=41)
    d = to_dev(c)
    inv = rope_inv_freq().to(DEV)
    b = len(lengths)
    ids = d["pos"].view(b, 1)
    q_r = ops.partial_rope(d["q"].unsqueeze(2), ids, inv, 64)[:, :, 0, :].contiguous()
    k_r = ops.partial_rope(d["k_new"].unsqueeze(2), ids, inv, 64)[:, :, 0, :].contiguous()
    kc1, vc1 = d["k_cache"].clone(), d["v_cache"].clone()
    ctx = ops.call_paged_gqa_attention_decode_triton(q_r, k_r, d["v_new"], kc1, vc1, d["block_table"], d["pos"])
    gate4 = d["gate"].view(b, 8, 256).permute(1, 0, 2).unsqueeze(0).contiguous()
    ctx4 = ctx.permute(1, 0, 2).unsqueeze(0).contiguous()
    chain = ops.attention_gate_pack(ctx4, gate4)
    kc2, vc2 = d["k_cache"].clone(), d["v_cache"].clone()
    fused = ops.fused_decode_attention(d["q"], d["k_new"], d["v_new"], d["gate"], kc2, vc2, d["block_table"], d["pos"],
                                       inv, 64, ops.fused_decode_workspace(DEV))
    assert torch.equal(kc1, kc2) and torch.equal(vc1, vc2)  # same rope arithmetic, same bytes in the cache
    assert maxabs(fused, chain) <= 2 ** -6


def test_decode_under_cuda_graph(ops):
    """Capture one step (fused kernel + in-graph pos += 1) and replay it 20 times; the page table already covers
    the growth.  Mirrors the reference's graph self-test (gqa_attention_decode.py:1133-1206)."""
    lengths = [30, 3, 200]
    steps = 20
    c = make_paged_case(lengths, seed=77, slack_tokens=steps + 4)
    inv = rope_inv_freq()
    d = to_dev(c)
    ws = ops.fused_decode_workspace(DEV)
    gen = torch.Generator().manual_seed(1)
    qs = [bf16_randn(3, 8, 256, gen=gen) for _ in range(steps)]
    ks = [bf16_randn(3, 2, 256, gen=gen) for _ in range(steps)]
    vs = [bf16_randn(3, 2, 256, gen=gen) for _ in range(steps)]
    q_s, k_s, v_s = d["q"].clone(), d["k_new"].clone(), d["v_new"].clone()
    pos = d["pos"].clone()
    out_s = torch.empty(3, 2048, dtype=torch.bfloat16, device=DEV)
    kc, vc = d["k_cache"].clone(), d["v_cache"].clone()
    pos0, kc0, vc0 = pos.clone(), kc.clone(), vc.clone()
    inv_d = inv.to(DEV)

    def step():
        ops.fused_decode_attention(q_s, k_s, v_s, d["gate"], kc, vc, d["block_table"], pos, inv_d, 64, ws, out=out_s)
        pos.add_(1)

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):
            step()
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    pos.copy_(pos0); kc.copy_(kc0); vc.copy_(vc0)   # capture and warm-up dirtied the state
    kr, vr = c["k_cache"].clone(), c["v_cache"].clone()
    p = c["pos"].clone()
    for i in range(steps):
        q_s.copy_(qs[i]); k_s.copy_(ks[i]); v_s.copy_(vs[i])
        graph.replay()
        ref = O.fused_decode_attention(qs[i], ks[i], vs[i], c["gate"], kr, vr, c["block_table"], p, inv, 64, exact=True)
        p += 1
        assert maxabs(out_s, ref) < TOL, f"step {i}"
    assert torch.equal(pos.cpu(), p)
    no_timeouts()


def test_overlapped_decode_attention_in_graph_equals_plain(ops):
    """projection -> q-norm -> k-norm -> fused decode attention in plain stream order, against projection -> fused decode
    attention with the head norms inside the kernel and the overlap flags set (it starts while the projection runs and
    requests its first pages before it waits), replayed from a CUDA graph with a new input every replay: outputs,
    caches and positions must be the same bytes.  A kernel that read the projection before it was complete would see
    the previous replay's values."""
    lengths = [30, 3, 200, 1025]
    steps = 6
    c = make_paged_case(lengths, seed=78, slack_tokens=steps + 4)
    d = to_dev(c)
    inv_d = rope_inv_freq().to(DEV)
    b = len(lengths)
    gen = torch.Generator().manual_seed(2)
    xs = [bf16_randn(b, 256, gen=gen).to(DEV) for _ in range(steps)]
    w = (torch.randn((8 + 8 + 2 + 2) * 256, 256, generator=gen) * 0.08).to(torch.bfloat16).to(DEV)
    qw = (torch.randn(256, generator=gen) * 0.1).to(torch.bfloat16).to(DEV)
    kw = (torch.randn(256, generator=gen) * 0.1).to(torch.bfloat16).to(DEV)

    def run(overlapped: bool):
        x = xs[0].clone()
        kc, vc, pos = d["k_cache"].clone(), d["v_cache"].clone(), d["pos"].clone()
        ws = ops.fused_decode_workspace(DEV)
        out = torch.empty(b, 2048, dtype=torch.bfloat16, device=DEV)

        def step():
            if overlapped:
                fused = ops.skinny_gemm(x, w, overlap=ops.OVERLAP_START | ops.OVERLAP_TRIGGER)
                ops.fused_decode_attention(fused[:, :2048].view(b, 8, 256), fused[:, 4096:4608].view(b, 2, 256),
                                           fused[:, 4608:].view(b, 2, 256), fused[:, 2048:4096], kc, vc,
                                           d["block_table"], pos, inv_d, 64, ws, out=out,
                                           overlap=ops.OVERLAP_START | ops.OVERLAP_PREFETCH,
                                           q_norm_weight=qw, k_norm_weight=kw, eps=1e-6)
            else:
                fused = ops.skinny_gemm(x, w)
                q = ops.add_rmsnorm(fused[:, :2048].view(b, 8, 256), qw, 1e-6)
                k = ops.add_rmsnorm(fused[:, 4096:4608].view(b, 2, 256), kw, 1e-6)
                ops.fused_decode_attention(q, k, fused[:, 4608:].view(b, 2, 256), fused[:, 2048:4096], kc, vc,
                                           d["block_table"], pos, inv_d, 64, ws, out=out)
            pos.add_(1)

        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            step()
        torch.cuda.current_stream().wait_stream(side)
        outs = [out.clone()]
        graph = None
        if overlapped:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                step()
            graph.replay()                       # the capture itself does not execute
        else:
            step()
        outs.append(out.clone())
        for nxt in xs[1:]:
            x.copy_(nxt)
            graph.replay() if graph is not None else step()
            outs.append(out.clone())
        torch.cuda.synchronize()
        return outs, kc, vc, pos

    plain, fast = run(False), run(True)
    no_timeouts()
    for x, y in zip(plain[0], fast[0]):
        assert torch.equal(x, y)
    assert torch.equal(plain[1], fast[1]) and torch.equal(plain[2], fast[2]) and torch.equal(plain[3], fast[3])


@pytest.mark.parametrize("one_launch", [False, True])
def test_chained_launches_change_nothing_but_time(ops, one_launch, monkeypatch):
    """The small decode-step operators are launched for programmatic dependent launch by default; the same chain with
    the switch off must give the same bytes (rope x2 -> append -> split -> combine -> gate-pack, or rope x2 -> the
    one-launch decode symbol -> gate-pack; three rounds so that every kernel also runs behind a kernel of its own
    kind)."""
    monkeypatch.setattr(ops, "DECODE_CALL_ONE_LAUNCH", one_launch)
    lengths = [700, 33, 2100, 512, 16, 1]
    c = make_paged_case(lengths, seed=77)
    inv = rope_inv_freq().to(DEV)
    d = to_dev(c)
    b = len(lengths)
    ids = d["pos"].view(b, 1)
    gate4 = d["gate"].view(b, 8, 256).permute(1, 0, 2).unsqueeze(0)

    def chain(k_cache, v_cache):
        outs = []
        for _ in range(3):
            q4 = ops.partial_rope(d["q"].unsqueeze(2), ids, inv, 64)
            k4 = ops.partial_rope(d["k_new"].unsqueeze(2), ids, inv, 64)
            ctx = ops.call_paged_gqa_attention_decode_triton(q4[:, :, 0, :], k4[:, :, 0, :], d["v_new"], k_cache, v_cache,
                                                             d["block_table"], d["pos"])
            outs.append(ops.attention_gate_pack(ctx.permute(1, 0, 2).unsqueeze(0), gate4))
        torch.cuda.synchronize()
        return outs

    kc1, vc1 = d["k_cache"].clone(), d["v_cache"].clone()
    chained = chain(kc1, vc1)
    ops.set_chain_overlap(False)
    try:
        kc2, vc2 = d["k_cache"].clone(), d["v_cache"].clone()
        plain = chain(kc2, vc2)
    finally:
        ops.set_chain_overlap(True)
    for a, p in zip(chained, plain):
        assert torch.equal(a, p)
    assert torch.equal(kc1, kc2) and torch.equal(vc1, vc2)
    no_timeouts()
