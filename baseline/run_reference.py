"""Runs the reference engine (the unmodified copy under baseline/_ref) on a GPU, with one of two operator sets:

    --kernels triton   the reference's own Triton kernels (its `triton_kernels/` package, JIT-compiled by the
                       installed Triton for the local GPU): the thing this repository replaces
    --kernels b200     this repository's drop-in `triton_kernels/` package (the CUDA library) under the SAME
                       reference `engine/runner.py`, `cache.py`, `paging.py`
    --kernels b200-fast  the same, with the opt-in `b200attn.fast_runner` subclass of the reference runner that takes
                       the fused decode / packed-prefill entry points

Both operator sets register the same `wy_lib::*` torch operators, so they cannot live in one process: a caller
(bench.py, the parity test) starts this script once per operator set and reads the result file.

Tasks (--task):
    parity       random-init model (seed 4) in the reference's own weight dataclasses, packed prefill of B prompts, then S
                 decode steps.  Without --teacher the steps are greedy; with --teacher <file of an earlier run> the
                 inputs of every step are that run's tokens ("teacher forcing"), so the two runs see identical inputs
                 at every step.  Writes tokens and the final hidden state of every step.
    model_bench  whole-model timing of the reference runner: packed prefill (ms) and S decode steps replayed from its
                 own CUDA graph (`GraphedDecoder`), device time.
    op_bench     device time of the reference operator chains at the benchmark shapes (decode attention layer step,
                 Gated-DeltaNet decode step, packed prefill attention, Gated-DeltaNet prefill), each replayed from a
                 CUDA graph.
    cpu_legs     no GPU: the reference's decode-attention path on the host cores, (a) its Triton operators executed by
                 the Triton interpreter (set TRITON_INTERPRET=1) on benchmark configuration 1, (b) its eager PyTorch
                 functions on a bounded sample of the headline workload.

Weights are synthetic: every tensor ~N(0, 0.02) in bf16 from one seeded generator (A_log ~ U(0, 2.7) and the gated-norm
weight 1 + N(0, 0.02) in fp32), laid out as `engine/loader.py` lays out a checkpoint (fused row blocks with row views).
No checkpoint, tokenizer or dataset is involved.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from pathlib import Path

HERE = Path(__file__).resolve().parent
REF = HERE / "_ref"
PKG = HERE.parent / "qwen3_5-triton-inference-engine_b200"

FULL = dict(hidden=1024, layers=24, vocab=248320, heads_q=8, heads_kv=2, head_dim=256, rotary_dim=64, rope_theta=1e7,
            gdn_heads=16, gdn_dim=128, intermediate=3584, eps=1e-6)


def setup_paths(kernels: str) -> None:
    """Make `import triton_kernels` resolve to the chosen operator set and `import engine` to the reference copy."""
    if not (REF / "engine" / "runner.py").exists():
        raise SystemExit(f"{REF} is absent: run `python baseline/make_ref.py` where the reference checkout is available")
    if kernels.startswith("b200"):
        sys.path.insert(0, str(PKG))
        import triton_kernels  # noqa: F401  this repository's drop-in; must be imported before the reference engine
        assert Path(triton_kernels.__file__).resolve().is_relative_to(PKG)
        sys.path.insert(1, str(REF))
    else:
        sys.path.insert(0, str(REF))


def random_tensors(cfg: dict, seed: int, device) -> dict:
    """Every parameter tensor of the architecture from ONE generator, in a fixed order (so that two processes on the
    same kind of device build bit-identical weights)."""
    import torch
    gen = torch.Generator(device=device).manual_seed(seed)

    def rnd(*shape, dtype=torch.bfloat16, std=0.02):
        return (torch.randn(*shape, generator=gen, device=device, dtype=torch.float32) * std).to(dtype)

    hid, inter = cfg["hidden"], cfg["intermediate"]
    kd = cfg["gdn_heads"] * cfg["gdn_dim"]
    qd, kvd = cfg["heads_q"] * cfg["head_dim"], cfg["heads_kv"] * cfg["head_dim"]
    out = {"embed": rnd(cfg["vocab"], hid), "norm": rnd(hid), "layers": []}
    for i in range(cfg["layers"]):
        layer = {"ln1": rnd(hid), "ln2": rnd(hid), "gate_up": rnd(2 * inter, hid), "down": rnd(hid, inter)}
        if (i + 1) % 4 == 0:   # full attention at layers 3, 7, 11, ...
            layer.update(kind="attention", qkvg=rnd(2 * qd + 2 * kvd, hid), q_norm=rnd(cfg["head_dim"]),
                         k_norm=rnd(cfg["head_dim"]), o_proj=rnd(hid, qd))
        else:
            layer.update(kind="gdn", in_proj=rnd(4 * kd + 2 * cfg["gdn_heads"], hid), conv=rnd(3 * kd, 4),
                         a_log=torch.rand(cfg["gdn_heads"], generator=gen, device=device) * 2.7,
                         dt_bias=rnd(cfg["gdn_heads"]), gdn_norm=1.0 + rnd(cfg["gdn_dim"], dtype=torch.float32),
                         out_proj=rnd(hid, kd))
        out["layers"].append(layer)
    return out


def text_weights(cfg: dict, tensors: dict):
    """The tensors in the reference's own frozen dataclasses (engine/loader.py:82-153), fused blocks with row views as
    `_fuse_rows` builds them (engine/loader.py:46-79)."""
    from engine import loader as L
    kd = cfg["gdn_heads"] * cfg["gdn_dim"]
    qd, kvd = cfg["heads_q"] * cfg["head_dim"], cfg["heads_kv"] * cfg["head_dim"]
    inter = cfg["intermediate"]
    layers = []
    for t in tensors["layers"]:
        gu = t["gate_up"]
        mlp = L.MLPWeights(gate_proj=gu[:inter], up_proj=gu[inter:], down_proj=t["down"], gate_up=gu)
        if t["kind"] == "gdn":
            f = t["in_proj"]
            h = cfg["gdn_heads"]
            layers.append(L.GDNLayerWeights(
                input_layernorm=t["ln1"], post_attention_layernorm=t["ln2"], in_proj_qkv=f[: 3 * kd],
                in_proj_z=f[3 * kd: 4 * kd], in_proj_a=f[4 * kd: 4 * kd + h], in_proj_b=f[4 * kd + h:], in_proj_fused=f,
                conv1d=t["conv"], conv1d_decode=t["conv"].t().contiguous(), a_log=t["a_log"], dt_bias=t["dt_bias"],
                norm=t["gdn_norm"], out_proj=t["out_proj"], mlp=mlp))
        else:
            f = t["qkvg"]
            layers.append(L.AttnLayerWeights(
                input_layernorm=t["ln1"], post_attention_layernorm=t["ln2"], q_proj_q=f[:qd], q_proj_gate=f[qd: 2 * qd],
                k_proj=f[2 * qd: 2 * qd + kvd], v_proj=f[2 * qd + kvd:], qkvg_fused=f, q_norm=t["q_norm"],
                k_norm=t["k_norm"], o_proj=t["o_proj"], mlp=mlp))
    return L.TextWeights(
        embed_tokens=tensors["embed"], norm=tensors["norm"], layers=tuple(layers), hidden_size=cfg["hidden"],
        num_layers=cfg["layers"], vocab_size=cfg["vocab"], rms_norm_eps=cfg["eps"], rope_theta=cfg["rope_theta"],
        rotary_dim=cfg["rotary_dim"], num_attention_heads=cfg["heads_q"], num_key_value_heads=cfg["heads_kv"],
        head_dim=cfg["head_dim"], linear_num_heads=cfg["gdn_heads"], linear_head_dim=cfg["gdn_dim"])


def runner_class(kernels: str):
    """The reference's `Qwen35Runner`, or this package's opt-in subclass of it."""
    if kernels == "b200-fast":
        from b200attn.fast_runner import fast_runner_class
        return fast_runner_class()
    from engine.runner import Qwen35Runner
    return Qwen35Runner


def make_prompts(cfg, batch, prompt_len, seed, ragged):
    import torch
    gen = torch.Generator().manual_seed(seed)
    lengths = [prompt_len] * batch
    if ragged:
        lengths = torch.randint(max(1, prompt_len // 4), prompt_len + 1, (batch,), generator=gen).tolist()
    return [torch.randint(0, cfg["vocab"], (n,), generator=gen, dtype=torch.int64) for n in lengths]


def events_ms(fn, repeat=1):
    import torch
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for _ in range(repeat):
        fn()
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) / repeat


# ----------------------------------------------------------------------------------------------------------- tasks
def task_parity(args, cfg):
    import torch
    from engine.cache import allocate_caches
    from triton_kernels.vocab_argmax import lm_head_argmax

    dev = torch.device("cuda", 0)
    w = text_weights(cfg, random_tensors(cfg, args.seed, dev))
    runner = runner_class(args.kernels)(w, compile=False)
    prompts = [p.to(dev) for p in make_prompts(cfg, args.batch, args.prompt_len, args.seed, args.ragged)]
    max_len = max(p.numel() for p in prompts) + args.steps + 8
    caches = allocate_caches(w, max_len, paged=True, batch=args.batch)
    caches.reset()
    teacher = torch.load(args.teacher)["tokens"].to(dev) if args.teacher else None
    hiddens, tokens = [], []
    last = torch.stack([h[-1] for h in runner.prefill_packed(prompts, caches)])          # [B, hidden]
    for step in range(args.steps + 1):
        hiddens.append(last)
        tok = lm_head_argmax(last.contiguous(), w.embed_tokens, last_only=False)
        tokens.append(tok)
        if step == args.steps:
            break
        feed = teacher[step] if teacher is not None else tok
        last = runner.decode_step(feed.to(torch.int32), caches)
        caches.pos.add_(1)
    torch.cuda.synchronize()
    torch.save({"tokens": torch.stack(tokens).cpu(), "hidden": torch.stack(hiddens).cpu(), "kernels": args.kernels,
                "lengths": [p.numel() for p in prompts]}, args.out)
    return {"task": "parity", "kernels": args.kernels, "steps": args.steps, "batch": args.batch}


def task_model_bench(args, cfg):
    import torch
    from engine.cache import allocate_caches
    from engine.runner import GraphedDecoder
    from triton_kernels.vocab_argmax import lm_head_argmax

    dev = torch.device("cuda", 0)
    w = text_weights(cfg, random_tensors(cfg, args.seed, dev))
    runner = runner_class(args.kernels)(w, compile=False)
    prompts = [p.to(dev) for p in make_prompts(cfg, args.batch, args.prompt_len, args.seed, False)]
    max_len = args.prompt_len + args.steps + 24
    caches = allocate_caches(w, max_len, paged=True, batch=args.batch)

    def prefill():
        caches.reset()
        hid = runner.prefill_packed(prompts, caches)
        return lm_head_argmax(torch.stack([h[-1] for h in hid]).contiguous(), w.embed_tokens, last_only=False)

    t0 = time.perf_counter()
    first = prefill()                  # JIT compilation + autotuning of every prefill kernel
    torch.cuda.synchronize()
    compile_s = time.perf_counter() - t0
    prefill()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    first = prefill()
    torch.cuda.synchronize()
    prefill_wall_ms = (time.perf_counter() - t0) * 1e3
    decoder = GraphedDecoder(runner, caches)
    decoder.tok_slot.copy_(first.to(torch.int32))
    t0 = time.perf_counter()
    decoder.capture()                  # warm-up steps (JIT + autotune of the decode kernels) and the capture
    torch.cuda.synchronize()
    capture_s = time.perf_counter() - t0
    first = prefill()                  # capture left the caches dirty
    decoder.tok_slot.copy_(first.to(torch.int32))
    torch.cuda.synchronize()
    ms = events_ms(decoder.graph.replay, repeat=args.steps)
    tokens = decoder.tok_out.tolist()
    return {"task": "model_bench", "kernels": args.kernels, "batch": args.batch, "prompt_len": args.prompt_len,
            "decode_steps": args.steps, "ms_per_step": ms, "tok_s": args.batch / (ms * 1e-3),
            "prefill_ms": prefill_wall_ms, "first_prefill_s": compile_s, "capture_s": capture_s,
            "last_tokens": tokens[:4]}


def graph_time(fn, steps, warm=3):
    """ms per call of `fn`, replayed `steps` times from one CUDA graph (device time, no Python dispatch)."""
    import torch
    for _ in range(warm):
        fn(0)
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(warm):
            fn(0)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(steps):
            fn(i)
    graph.replay()
    torch.cuda.synchronize()
    return events_ms(graph.replay) / steps


def task_op_bench(args, cfg):
    """The reference's operator chains at the benchmark shapes.  Rotating copies of the big operands keep L2 from
    serving a call what the previous call loaded (the 126 MB L2 holds none of these working sets three times)."""
    import torch
    import torch.nn.functional as F
    from triton_kernels.attention_gate_pack import attention_gate_pack
    from triton_kernels.gdn_recurrent_prefill import (call_gdn_recurrent_prefill_chunked_triton, gdn_recurrent_decode,
                                                      gdn_recurrent_prefill_sequential)
    from triton_kernels.gqa_attention_decode_paged import (allocate_split_scratch, call_paged_gqa_attention_decode_triton,
                                                           paged_kv_fill_varlen)
    from triton_kernels.gqa_attention_varlen_causal import build_cu_seqlens, gqa_attention_varlen_causal
    from triton_kernels.partial_rope import partial_rope

    dev = torch.device("cuda", 0)
    hq, hkv, d, rot, page = 8, 2, 256, 64, 16
    inv = (1.0 / (1e7 ** (torch.arange(0, rot, 2, dtype=torch.float32) / rot))).to(dev)
    l2 = 126 * 1024 * 1024
    rows = []
    steps = args.steps
    batches = [int(b) for b in args.batches.split(",")]
    for mode in (("random",) if args.only == "decode_random" else ("random", "fixed32768")):
        for b in batches:
            if mode == "fixed32768" and b > 32:
                continue
            gen = torch.Generator().manual_seed(1)
            lengths = [32768] * b if mode == "fixed32768" else torch.randint(512, 4097, (b,), generator=gen).tolist()
            pps = [(n + 1 + page - 1) // page for n in lengths]
            nbytes = sum(2048 * (n + 1) for n in lengths)
            sets = max(1, min(16, -(-3 * l2 // nbytes)))
            num_pages = sum(pps) + 8
            tables, kcs, vcs = [], [], []
            for _ in range(sets):
                perm = torch.randperm(num_pages, generator=gen)
                table = torch.zeros(b, max(pps), dtype=torch.int32)
                off = 0
                for i, n in enumerate(pps):
                    table[i, :n] = perm[off:off + n].to(torch.int32)
                    off += n
                tables.append(table.to(dev))
                kcs.append(torch.randn(num_pages, hkv, page, d, dtype=torch.bfloat16, device=dev))
                vcs.append(torch.randn(num_pages, hkv, page, d, dtype=torch.bfloat16, device=dev))
            q = torch.randn(b, hq, d, dtype=torch.bfloat16, device=dev)
            kn = torch.randn(b, hkv, d, dtype=torch.bfloat16, device=dev)
            vn = torch.randn(b, hkv, d, dtype=torch.bfloat16, device=dev)
            gate = torch.randn(b, hq * d, dtype=torch.bfloat16, device=dev)
            pos = torch.tensor(lengths, dtype=torch.int64, device=dev)
            ids = pos.view(b, 1)
            scratch = allocate_split_scratch(hq, d, batch=b, device=dev)

            def chain(i):   # engine/runner.py:482-517 without the projections and head norms
                s = i % sets
                q4 = partial_rope(q.unsqueeze(2), ids, inv, rot)
                k4 = partial_rope(kn.unsqueeze(2), ids, inv, rot)
                ctx = call_paged_gqa_attention_decode_triton(q4[:, :, 0, :].contiguous(), k4[:, :, 0, :].contiguous(), vn,
                                                             kcs[s], vcs[s], tables[s], pos, scratch)
                gate4 = gate.view(b, hq, d).permute(1, 0, 2).unsqueeze(0).contiguous()
                return attention_gate_pack(ctx.permute(1, 0, 2).unsqueeze(0).contiguous(), gate4)

            ms = graph_time(chain, steps)
            rows.append({"op": "decode_chain", "B": b, "ctx": mode, "us": ms * 1e3})
            del tables, kcs, vcs
            torch.cuda.empty_cache()
    if args.only == "decode_random":
        return {"task": "op_bench", "kernels": args.kernels, "rows": rows}
    # Gated-DeltaNet decode step
    for b in (1, 32, 256):
        nbytes = b * 2 * 16 * 128 * 128 * 4
        sets = max(1, min(32, -(-3 * l2 // nbytes)))
        states = [torch.zeros(b, 16, 128, 128, device=dev) for _ in range(sets)]
        gen = torch.Generator().manual_seed(3)
        gq = F.normalize(torch.randn(b, 16, 128, generator=gen), dim=-1).to(torch.bfloat16).to(dev)
        gk = F.normalize(torch.randn(b, 16, 128, generator=gen), dim=-1).to(torch.bfloat16).to(dev)
        gv = torch.randn(b, 16, 128, generator=gen).to(torch.bfloat16).to(dev)
        beta = torch.sigmoid(torch.randn(b, 16, generator=gen)).to(dev)
        g = (-F.softplus(torch.randn(b, 16, generator=gen))).to(dev)
        ms = graph_time(lambda i: gdn_recurrent_decode(gq, gk, gv, beta, g, states[i % sets]), steps)
        rows.append({"op": "gdn_recurrent_decode", "B": b, "us": ms * 1e3})
        del states
        torch.cuda.empty_cache()
    # packed prefill attention: the benchmark's B=32 draw and a long-prompt shape
    gen = torch.Generator().manual_seed(2)
    for tag, lengths in (("cfg3 B=32 L~U[16,512]", torch.randint(16, 513, (32,), generator=gen).tolist()),
                         ("long B=8 L=4096", [4096] * 8)):
        total = sum(lengths)
        q = torch.randn(total, hq, d, device=dev, dtype=torch.bfloat16)
        k = torch.randn(total, hkv, d, device=dev, dtype=torch.bfloat16)
        v = torch.randn(total, hkv, d, device=dev, dtype=torch.bfloat16)
        gate = torch.randn(total, hq * d, device=dev, dtype=torch.bfloat16)
        cu, max_len = build_cu_seqlens(lengths, device=dev)
        ms = graph_time(lambda i: gqa_attention_varlen_causal(q, k, v, cu, max_len), steps)
        rows.append({"op": "gqa_attention_varlen_causal", "shape": tag, "us": ms * 1e3})
        pps = [(n + page - 1) // page for n in lengths]
        table = torch.zeros(len(lengths), max(pps), dtype=torch.int32)
        perm = torch.randperm(sum(pps), generator=gen)
        off = 0
        for i, n in enumerate(pps):
            table[i, :n] = perm[off:off + n].to(torch.int32)
            off += n
        table = table.to(dev)
        kc = torch.zeros(sum(pps), hkv, page, d, dtype=torch.bfloat16, device=dev)
        vc = torch.zeros_like(kc)
        ids = torch.cat([torch.arange(n) for n in lengths]).to(torch.int32).to(dev).unsqueeze(0)

        def layer(i):   # engine/runner.py:339-384 without the projections and head norms
            q4 = partial_rope(q.unsqueeze(0).permute(0, 2, 1, 3), ids, inv, rot)
            k4 = partial_rope(k.unsqueeze(0).permute(0, 2, 1, 3), ids, inv, rot)
            v4 = v.unsqueeze(0).permute(0, 2, 1, 3)
            ctx = gqa_attention_varlen_causal(q4[0].permute(1, 0, 2).contiguous(), k4[0].permute(1, 0, 2).contiguous(),
                                              v4[0].permute(1, 0, 2).contiguous(), cu, max_len)
            out = attention_gate_pack(ctx.permute(1, 0, 2).unsqueeze(0), gate.view(1, total, hq, d).permute(0, 2, 1, 3))
            paged_kv_fill_varlen(kc, vc, k4[0], v4[0], table, cu, max_len)
            return out

        ms = graph_time(layer, steps)
        rows.append({"op": "prefill_attention_layer_chain", "shape": tag, "us": ms * 1e3})
        del q, k, v, gate, kc, vc
        torch.cuda.empty_cache()
    # Gated-DeltaNet prefill: the packed benchmark shape (the reference's only packed route is token-serial) and the
    # single-sequence chunk-64 pipeline at T = 2048
    heads = 16
    for tag, lengths in (("cfg4 B=32 x 128", [128] * 32), ("1 x 2048", [2048])):
        total = sum(lengths)
        gen = torch.Generator().manual_seed(3)
        gq = (F.normalize(torch.randn(total, heads, 128, generator=gen), dim=-1) * 128 ** -0.5).to(torch.bfloat16).to(dev)
        gk = F.normalize(torch.randn(total, heads, 128, generator=gen), dim=-1).to(torch.bfloat16).to(dev)
        gv = torch.randn(total, heads, 128, generator=gen).to(torch.bfloat16).to(dev)
        beta = torch.sigmoid(torch.randn(total, heads, generator=gen)).to(dev)
        g = (-F.softplus(torch.randn(total, heads, generator=gen)) * torch.exp(torch.rand(heads, generator=gen) * 2.7)).to(dev)
        cu, _ = build_cu_seqlens(lengths, device=dev)
        # the operator reads cu_seqlens[-1] on the host (an assert), which a CUDA graph cannot hold: time it eagerly,
        # many calls between two events, after a warm-up
        for _ in range(3):
            gdn_recurrent_prefill_sequential(gq, gk, gv, beta, g, cu)
        ms = events_ms(lambda: gdn_recurrent_prefill_sequential(gq, gk, gv, beta, g, cu), repeat=max(4, steps // 2))
        rows.append({"op": "gdn_recurrent_prefill_sequential", "shape": tag, "us": ms * 1e3, "timing": "eager loop"})
        if len(lengths) == 1:
            ms = graph_time(lambda i: call_gdn_recurrent_prefill_chunked_triton(gq, gk, gv, beta, g), max(2, steps // 4))
            rows.append({"op": "gdn chunk-64 pipeline (3 launches)", "shape": tag, "us": ms * 1e3})
    return {"task": "op_bench", "kernels": args.kernels, "rows": rows}


def task_cpu_legs(args, cfg):
    """The two CPU baselines of the decode-attention path, run on the host cores with the reference's own code:
    (a) benchmark configuration 1 (B=4, contexts [37,64,100,128], seed 0) through the reference's Triton operators
        executed by the Triton interpreter (TRITON_INTERPRET=1 must be set by the caller; single-threaded Python);
    (b) one decode-attention layer step of the headline workload (first `--batch` sequences of the B=256 draw) through
        the reference's eager PyTorch functions (`partial_rope._torch_reference`, `torch_paged_reference`,
        `attention_gate_pack._torch_reference`), all host threads."""
    import torch
    hq, hkv, d, rot, page = 8, 2, 256, 64, 16
    out = {"task": "cpu_legs", "host_cores": os.cpu_count(), "torch_threads": torch.get_num_threads()}
    if os.environ.get("TRITON_INTERPRET") == "1" and not args.skip_interpreter:
        import importlib.util
        spec = importlib.util.spec_from_file_location("interpreter_shims", HERE / "interpreter_shims.py")
        shims = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(shims)
        pin = shims.install_shims()
        from triton_kernels import gqa_attention_decode_paged as ref
        pin()
        torch.manual_seed(0)
        lens = [37, 64, 100, 128]
        batch = len(lens)
        pps = (128 + page - 1) // page + 1
        num_pages = batch * pps
        table = torch.randperm(num_pages)[: batch * pps].view(batch, pps).int()
        kc = torch.randn(num_pages, hkv, page, d).to(torch.bfloat16)
        vc = torch.randn(num_pages, hkv, page, d).to(torch.bfloat16)
        q = torch.randn(batch, hq, d).to(torch.bfloat16)
        kn = torch.randn(batch, hkv, d).to(torch.bfloat16)
        vn = torch.randn(batch, hkv, d).to(torch.bfloat16)
        pos = torch.tensor([n - 1 for n in lens], dtype=torch.int64)
        scratch = ref.allocate_split_scratch(hq, d, batch=batch, device="cpu")
        t0 = time.perf_counter()
        got = ref.call_paged_gqa_attention_decode_triton(q, kn, vn, kc, vc, table, pos, scratch)
        interp_s = time.perf_counter() - t0
        t0 = time.perf_counter()
        want = ref.torch_paged_reference(q, kc, vc, table, lens)
        eager_s = time.perf_counter() - t0
        out["interpreter"] = {"workload": "config 1: B=4, contexts [37,64,100,128], seed 0", "seconds": interp_s,
                              "effective_cores": 1, "eager_cpu_seconds": eager_s,
                              "max_abs_vs_eager": (got.float() - want.float()).abs().max().item()}
    # (b) eager CPU chain on a bounded sample of the headline workload
    from triton_kernels import attention_gate_pack as gp
    from triton_kernels import gqa_attention_decode_paged as ref
    from triton_kernels import partial_rope as pr
    gen = torch.Generator().manual_seed(1)
    lengths = torch.randint(512, 4097, (256,), generator=gen).tolist()[: args.batch]
    b = len(lengths)
    pps = [(n + 1 + page - 1) // page for n in lengths]
    num_pages = sum(pps) + 8
    perm = torch.randperm(num_pages, generator=gen)
    table = torch.zeros(b, max(pps), dtype=torch.int32)
    off = 0
    for i, n in enumerate(pps):
        table[i, :n] = perm[off:off + n].to(torch.int32)
        off += n
    kc = torch.randn(num_pages, hkv, page, d, generator=gen).to(torch.bfloat16)
    vc = torch.randn(num_pages, hkv, page, d, generator=gen).to(torch.bfloat16)
    q = torch.randn(b, hq, d, generator=gen).to(torch.bfloat16)
    kn = torch.randn(b, hkv, d, generator=gen).to(torch.bfloat16)
    vn = torch.randn(b, hkv, d, generator=gen).to(torch.bfloat16)
    gate = torch.randn(b, hq * d, generator=gen).to(torch.bfloat16)
    pos = torch.tensor(lengths, dtype=torch.int64)
    inv = 1.0 / (1e7 ** (torch.arange(0, rot, 2, dtype=torch.float32) / rot))
    ids = pos.view(b, 1)
    nbytes = (sum(2048 * (n + 1) for n in lengths) + b * (4096 + 4096 + 4096 + 2048 + 2048)
              + sum(4 * p_ for p_ in pps) + 8 * b)

    def step():
        q4 = pr._torch_reference(q.unsqueeze(2), ids, inv, rot)
        k4 = pr._torch_reference(kn.unsqueeze(2), ids, inv, rot)
        for i, n in enumerate(lengths):                       # the reference's append operator exists for CUDA only
            phys = int(table[i, n // page])
            kc[phys, :, n % page] = k4[i, :, 0]
            vc[phys, :, n % page] = vn[i]
        ctx = ref.torch_paged_reference(q4[:, :, 0, :], kc, vc, table, [n + 1 for n in lengths])
        g4 = gate.view(b, hq, d).permute(1, 0, 2).unsqueeze(0)
        return gp._torch_reference(ctx.to(torch.bfloat16).permute(1, 0, 2).unsqueeze(0), g4)

    step()
    times = []
    t_end = time.time() + 20
    while len(times) < args.steps and (time.time() < t_end or not times):
        t0 = time.perf_counter()
        step()
        times.append(time.perf_counter() - t0)
    sec = sum(times) / len(times)
    out["eager_cpu"] = {"seconds_per_step": sec, "bytes_per_step": nbytes, "gbs": nbytes / sec / 1e9, "sequences": b,
                        "passes": len(times), "cores": torch.get_num_threads()}
    return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernels", choices=["triton", "b200", "b200-fast"], required=True)
    ap.add_argument("--task", choices=["parity", "model_bench", "op_bench", "cpu_legs"], required=True)
    ap.add_argument("--out", required=True, help="result file: .pt for parity, .json otherwise")
    ap.add_argument("--teacher", default=None)
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--prompt-len", type=int, default=32)
    ap.add_argument("--steps", type=int, default=16)
    ap.add_argument("--seed", type=int, default=4)
    ap.add_argument("--ragged", action="store_true", help="parity: prompt lengths drawn in [prompt_len/4, prompt_len]")
    ap.add_argument("--layers", type=int, default=FULL["layers"])
    ap.add_argument("--vocab", type=int, default=FULL["vocab"])
    ap.add_argument("--batches", default="1,4,16,32,64,256")
    ap.add_argument("--skip-interpreter", action="store_true")
    ap.add_argument("--only", default="all", choices=["all", "decode_random"], help="op_bench: which rows to run")
    args = ap.parse_args()
    setup_paths(args.kernels)
    import torch
    if args.task == "cpu_legs":
        try:   # launchers export OMP_NUM_THREADS=1; the CPU baseline is meant to use every host core it can
            torch.set_num_threads(max(1, len(os.sched_getaffinity(0))))
        except Exception:
            pass
    else:
        if not torch.cuda.is_available():
            raise SystemExit("this task needs a CUDA device")
        torch.cuda.set_device(0)
    cfg = dict(FULL, layers=args.layers, vocab=args.vocab)
    t0 = time.perf_counter()
    with torch.no_grad():
        result = {"parity": task_parity, "model_bench": task_model_bench, "op_bench": task_op_bench,
                  "cpu_legs": task_cpu_legs}[args.task](args, cfg)
    result["wall_s"] = time.perf_counter() - t0
    result["triton"] = __import__("triton").__version__ if args.kernels == "triton" else None
    if args.task == "parity":
        print(json.dumps(result))
    else:
        Path(args.out).write_text(json.dumps(result))
        print(json.dumps(result))


if __name__ == "__main__":
    os.environ.setdefault("TRITON_CACHE_AUTOTUNING", "1")
    main()
