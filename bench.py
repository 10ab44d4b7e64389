#!/usr/bin/env python
"""Benchmark of the attention hot path on B200: one full-attention layer decode step.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--batch B] [--no-sweep] [--impl reference|reference-triton]

A step = one launch of the fused decode-attention kernel (partial RoPE on q/k, KV append, paged GQA attention with
split-K over pages, sigmoid gate) over a batch of B sequences with contexts drawn uniform in [512, 4096] (seed 1):
8 Q heads, 2 KV heads, head_dim 256, 16-token pages, random page table, bf16 ~N(0,1) data, RoPE on the first 64 dims
with theta 1e7.  Synthetic data throughout.

Reported on one JSON line:
  value      achieved HBM GB/s = ALGORITHMIC bytes per step / device time (CUDA events), inputs resident in HBM
  e2e        same metric through the public Python operator with HOST inputs: per step q/k_new/v_new/gate are copied
             from pinned host memory and the [B,2048] output is copied back (the KV cache is device-resident state,
             as it is in the engine)
  roofline   the fused kernel against the measured copy bandwidth of this pool's B200s
  cpu_baseline  the reference's decode-attention path on the host cores: its eager PyTorch functions on a bounded sample
             of the workload (`value`), and its Triton operators under the Triton interpreter on the small CPU
             configuration (`interpreter`).  Without the reference copy (baseline/_ref) the oracle port is timed instead.
  sweep      us/layer and GB/s for B in {1,4,16,32,64,256}, random and fixed-32768 contexts, plus the drop-in
             3-launch chain, the Gated-DeltaNet decode state update, the decode-step projections and LM head of the
             whole model (cuBLAS time beside each) and the prefill operators (not part of `value`); `triton_us` beside a
             row is the reference's own Triton operator chain for the same shape on the same GPU
  reference_triton  the reference's Triton kernels on this GPU: the headline step, and its runner on the whole-model
             workload (on its own kernels, and unchanged on this package's drop-in operators)
`--impl reference` times the reference's CPU path (above) on a bounded sample of the same workload; `--impl
reference-triton` times the reference's Triton operator chain for the same step on the GPU.  Both need baseline/_ref
(`python baseline/make_ref.py`); without it the CPU arm falls back to the oracle port and the Triton arm prints an
`unavailable` line.
Under torchrun each rank runs its own replica (weak scaling, no data-path collective); the time is the max over ranks.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
PKG = ROOT / "qwen3_5-triton-inference-engine_b200"
for _p in (str(ROOT), str(PKG)):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import torch  # noqa: E402

PAGE, HQ, HKV, D, ROT = 16, 8, 2, 256, 64
L2_BYTES = 126 * 1024 * 1024
METRIC = "paged_gqa_decode_attention_hbm_gbs"
FALLBACK_HBM_GBS = 6650.0
# DRAM bytes / algorithmic bytes of the fused kernel in a profiler capture of the headline launch
# (1.2248 GB moved for 1.2143 GB algorithmic); the run itself does not measure DRAM traffic
NCU_TRAFFIC_RATIO = 1.009
REFERENCE_SCRIPT = ROOT / "baseline" / "run_reference.py"
REFERENCE_COPY = ROOT / "baseline" / "_ref"


def workload_config(batch: int) -> dict:
    """`config` of the JSON line, identical for every arm that measures this workload."""
    return {"workload": f"decode attention layer step, B={batch} per GPU, ctx~U[512,4096] seed 1, 8q/2kv heads, d=256, "
                        f"page 16, rope 64 theta 1e7, sigmoid gate",
            "l2_policy": "inputs larger than L2: every step streams its own KV pages (1.2 GB at B=256); smaller sweep "
                         "rows rotate over cache sets that together exceed three times L2"}


def run_reference_task(task: str, kernels: str, extra: list, timeout: int, env_extra: dict | None = None):
    """One run of baseline/run_reference.py in a child process (the reference's operators register the same torch
    operator names as this package's, so the two cannot share a process).  Returns (result dict or None, reason)."""
    if not (REFERENCE_COPY / "engine" / "runner.py").exists():
        return None, "baseline/_ref is absent (python baseline/make_ref.py copies the reference there)"
    fd, out = tempfile.mkstemp(suffix=".json")
    os.close(fd)
    env = dict(os.environ)
    for k in ("RANK", "LOCAL_RANK", "WORLD_SIZE", "MASTER_ADDR", "MASTER_PORT", "OMP_NUM_THREADS"):
        env.pop(k, None)
    env.update(env_extra or {})
    cmd = [sys.executable, str(REFERENCE_SCRIPT), "--kernels", kernels, "--task", task, "--out", out] + extra
    try:
        res = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env)
        if res.returncode != 0:
            tail = (res.stderr.strip().splitlines() or ["no output"])[-1]
            return None, f"{task} ({kernels}) exited {res.returncode}: {tail[:300]}"
        return json.loads(Path(out).read_text()), None
    except subprocess.TimeoutExpired:
        return None, f"{task} ({kernels}) did not finish in {timeout} s"
    except Exception as exc:  # unreadable result file
        return None, f"{task} ({kernels}): {exc}"
    finally:
        try:
            os.unlink(out)
        except OSError:
            pass


def cdiv(a, b):
    return (a + b - 1) // b


def draw_lengths(batch: int, mode: str, seed: int = 1) -> list[int]:
    if mode == "fixed32768":
        return [32768] * batch
    gen = torch.Generator().manual_seed(seed)
    return torch.randint(512, 4097, (batch,), generator=gen).tolist()


def algorithmic_bytes(lengths: list[int]) -> int:
    """K+V rows of every cached token incl. the appended one, q/gate/out rows, new-kv read + cache write,
    page-table entries and positions.  Split-K scratch is NOT algorithmic."""
    b = len(lengths)
    return (sum(2048 * (n + 1) for n in lengths) + b * (4096 + 4096 + 4096 + 2048 + 2048)
            + sum(4 * cdiv(n + 1, PAGE) for n in lengths) + 8 * b)


def gdn_decode_bytes(batch: int, heads: int = 16) -> int:
    return batch * (2 * heads * 128 * 128 * 4 + 3 * heads * 128 * 2 + heads * 128 * 2 + 2 * heads * 4)


class Workload:
    """`sets` independent copies of the layer state so that consecutive timed steps never find their pages in L2."""

    def __init__(self, lengths, device, seed=1, min_total_bytes=3 * L2_BYTES, max_sets=64, pin_host=False):
        self.lengths = lengths
        self.batch = b = len(lengths)
        self.device = device
        self.bytes = algorithmic_bytes(lengths)
        self.sets = max(1, min(max_sets, cdiv(min_total_bytes, self.bytes)))
        gen = torch.Generator().manual_seed(seed)
        pages_per_seq = [cdiv(n + 1, PAGE) for n in lengths]
        max_pages = max(pages_per_seq)
        used = sum(pages_per_seq)
        num_pages = used + 8
        self.inv_freq = (1.0 / (1e7 ** (torch.arange(0, ROT, 2, dtype=torch.float32) / ROT))).to(device)
        self.pos = torch.tensor(lengths, dtype=torch.int64, device=device)
        self.k_caches, self.v_caches, self.tables = [], [], []
        for _ in range(self.sets):
            perm = torch.randperm(num_pages, generator=gen)
            table = torch.zeros(b, max_pages, dtype=torch.int32)
            off = 0
            for i, n in enumerate(pages_per_seq):
                table[i, :n] = perm[off:off + n].to(torch.int32)
                off += n
            self.tables.append(table.to(device))
            self.k_caches.append(torch.randn(num_pages, HKV, PAGE, D, dtype=torch.bfloat16, device=device))
            self.v_caches.append(torch.randn(num_pages, HKV, PAGE, D, dtype=torch.bfloat16, device=device))
        host = dict(
            q=torch.randn(b, HQ, D, generator=gen).to(torch.bfloat16),
            k_new=torch.randn(b, HKV, D, generator=gen).to(torch.bfloat16),
            v_new=torch.randn(b, HKV, D, generator=gen).to(torch.bfloat16),
            gate=torch.randn(b, HQ * D, generator=gen).to(torch.bfloat16),
        )
        self.host = {k: (v.pin_memory() if pin_host else v) for k, v in host.items()}
        self.dev = {k: v.to(device) for k, v in host.items()}
        self.out = torch.empty(b, HQ * D, dtype=torch.bfloat16, device=device)
        self.out_host = torch.empty(b, HQ * D, dtype=torch.bfloat16).pin_memory() if pin_host else None


def capture_steps(fn, steps: int, first: int = 0):
    """One CUDA graph holding `steps` consecutive steps (step index first..first+steps-1), the way the engine runs
    decode: no host work between launches."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        fn(first)  # lazy initialisation (function attributes, allocator) must not happen under capture
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(steps):
            fn(first + i)
    return graph


def time_steps(fn, steps: int, warmup: int, use_graph: bool = True) -> float:
    """ms per step with CUDA events on the current (launching) stream; by default the `steps` launches are replayed
    from one CUDA graph so that the number is device time, not Python dispatch time."""
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if use_graph:
        graph = capture_steps(fn, steps, warmup)
        graph.replay()  # warm replay (graph upload)
        torch.cuda.synchronize()
        start.record()
        graph.replay()
        end.record()
    else:
        start.record()
        for i in range(steps):
            fn(warmup + i)
        end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) / steps


def fused_step(ops, w: Workload, ws):
    d = w.dev

    def fn(i):
        s = i % w.sets
        ops.fused_decode_attention(d["q"], d["k_new"], d["v_new"], d["gate"], w.k_caches[s], w.v_caches[s], w.tables[s],
                                   w.pos, w.inv_freq, ROT, ws, out=w.out)
    return fn


def chain_step(ops, w: Workload, scratch):
    """The operator calls of the reference runner's decode attention with our drop-in operators: rope x2, the decode
    symbol `call_paged_gqa_attention_decode_triton` (one launch by default; append, split, combine with
    ops.DECODE_CALL_ONE_LAUNCH off), gate-pack."""
    d = w.dev
    b = w.batch
    ids = w.pos.view(b, 1)

    def fn(i):
        s = i % w.sets
        q4 = ops.partial_rope(d["q"].unsqueeze(2), ids, w.inv_freq, ROT)
        k4 = ops.partial_rope(d["k_new"].unsqueeze(2), ids, w.inv_freq, ROT)
        ctx = ops.call_paged_gqa_attention_decode_triton(q4[:, :, 0, :], k4[:, :, 0, :], d["v_new"], w.k_caches[s],
                                                         w.v_caches[s], w.tables[s], w.pos, scratch)
        gate4 = d["gate"].view(b, HQ, D).permute(1, 0, 2).unsqueeze(0)
        ops.attention_gate_pack(ctx.permute(1, 0, 2).unsqueeze(0), gate4)
    return fn


def e2e_step(ops, w: Workload, ws):
    """One layer step the way a host drives the public operator: this step's q / k_new / v_new / gate come from pinned
    host memory and its [B, 2048] result goes back to pinned host memory, every step.  The copies run on two side
    streams with double-buffered device and host buffers, so that step i+1's inputs travel while step i computes
    (events order copy -> kernel -> copy-back per step and protect buffer reuse)."""
    h = w.host
    dev = w.device
    compute = torch.cuda.current_stream(dev)
    h2d, d2h = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    names = ("q", "k_new", "v_new", "gate")
    bufs = [{n: torch.empty_like(h[n], device=dev) for n in names} for _ in range(2)]
    outs = [torch.empty(w.out_host.shape, dtype=w.out_host.dtype, device=dev) for _ in range(2)]
    out_host = [w.out_host, torch.empty_like(w.out_host).pin_memory()]
    computed = [None, None]      # event: the kernel that read bufs[p] / wrote outs[p] is done
    drained = [None, None]       # event: outs[p] has been copied back

    def fn(i):
        p, s = i & 1, i % w.sets
        with torch.cuda.stream(h2d):
            if computed[p] is not None:
                h2d.wait_event(computed[p])
            for n in names:
                bufs[p][n].copy_(h[n], non_blocking=True)
            arrived = torch.cuda.Event()
            arrived.record(h2d)
        compute.wait_event(arrived)
        if drained[p] is not None:
            compute.wait_event(drained[p])
        b = bufs[p]
        ops.fused_decode_attention(b["q"], b["k_new"], b["v_new"], b["gate"], w.k_caches[s], w.v_caches[s], w.tables[s],
                                   w.pos, w.inv_freq, ROT, ws, out=outs[p])
        computed[p] = torch.cuda.Event()
        computed[p].record(compute)
        with torch.cuda.stream(d2h):
            d2h.wait_event(computed[p])
            out_host[p].copy_(outs[p], non_blocking=True)
            drained[p] = torch.cuda.Event()
            drained[p].record(d2h)
    return fn


# --------------------------------------------------------------------------- CPU oracle timing
def cpu_reference_step(lengths, sample: int, seed: int = 1):
    """Returns (seconds, algorithmic bytes) of one oracle pass over the first `sample` sequences of the workload."""
    from oracle import reference_ops as O

    lens = lengths[:sample]
    gen = torch.Generator().manual_seed(seed)
    b = len(lens)
    pps = [cdiv(n + 1, PAGE) for n in lens]
    num_pages = sum(pps) + 8
    perm = torch.randperm(num_pages, generator=gen)
    table = torch.zeros(b, max(pps), dtype=torch.int32)
    off = 0
    for i, n in enumerate(pps):
        table[i, :n] = perm[off:off + n].to(torch.int32)
        off += n
    kc = torch.randn(num_pages, HKV, PAGE, D, generator=gen).to(torch.bfloat16)
    vc = torch.randn(num_pages, HKV, PAGE, D, generator=gen).to(torch.bfloat16)
    q = torch.randn(b, HQ, D, generator=gen).to(torch.bfloat16)
    kn = torch.randn(b, HKV, D, generator=gen).to(torch.bfloat16)
    vn = torch.randn(b, HKV, D, generator=gen).to(torch.bfloat16)
    gate = torch.randn(b, HQ * D, generator=gen).to(torch.bfloat16)
    pos = torch.tensor(lens, dtype=torch.int64)
    inv = 1.0 / (1e7 ** (torch.arange(0, ROT, 2, dtype=torch.float32) / ROT))
    t0 = time.perf_counter()
    O.fused_decode_attention(q, kn, vn, gate, kc, vc, table, pos, inv, ROT, exact=True)
    return time.perf_counter() - t0, algorithmic_bytes(lens)


# --------------------------------------------------------------------------- clocks
class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.path = None

    def __enter__(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu_index)], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None
        return self

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()

    def summary(self) -> dict:
        sm, mx, reasons = [], [], set()
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 9:
                    continue
                sm.append(float(f[1]))
                mx.append(float(f[2]))
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def hbm_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


# --------------------------------------------------------------------------- main
def aggregate_over_ranks(ms_local: float, units_local: float, dist, device):
    """Whole-job figures of a replicated run: (slowest rank's time, units summed over ranks).  `dist` is
    torch.distributed (initialised) or None for a single process."""
    if dist is None:
        return ms_local, units_local
    t = torch.tensor([ms_local], device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    u = torch.tensor([units_local], device=device, dtype=torch.float64)
    dist.all_reduce(u, op=dist.ReduceOp.SUM)
    return float(t.item()), float(u.item())


def cpu_baseline_legs(batch: int, sample: int, passes: int):
    """The `cpu_baseline` object: the reference's own CPU code when its copy is present (eager PyTorch functions on the
    first `sample` sequences; Triton operators under the interpreter on configuration 1), else the oracle port."""
    legs, why = run_reference_task("cpu_legs", "triton", ["--batch", str(sample), "--steps", str(passes)], 240,
                                   {"TRITON_INTERPRET": "1"})
    if legs is not None:
        e = legs["eager_cpu"]
        base = {"value": e["gbs"], "unit": "GB/s", "cores": e["cores"], "kind": "reference",
                "sample": f"first {e['sequences']} of {batch} sequences, {e['passes']} passes, the reference's eager PyTorch "
                          f"functions (partial_rope, torch_paged_reference, attention_gate_pack) on the host",
                "seconds_per_step": e["seconds_per_step"]}
        if "interpreter" in legs:
            base["interpreter"] = dict(legs["interpreter"], host_cores=legs["host_cores"])
        return base, e["seconds_per_step"]
    lengths = draw_lengths(batch, "random")
    cpu_reference_step(lengths, min(sample, 8))
    secs, nbytes = [], 0
    t_budget = time.time() + 20
    while len(secs) < passes and (time.time() < t_budget or not secs):
        sec, nbytes = cpu_reference_step(lengths, sample)
        secs.append(sec)
    sec = sum(secs) / len(secs)
    return ({"value": nbytes / sec / 1e9, "unit": "GB/s", "cores": torch.get_num_threads(), "kind": "port",
             "sample": f"first {sample} of {batch} sequences, {len(secs)} passes, oracle port (eager PyTorch fp32); "
                       f"reference copy unavailable: {why}"}, sec)


def run_reference(args, rank, world):
    """`--impl reference`: the reference's CPU path for the same step, on the host cores (rank 0 only)."""
    if rank != 0:
        return
    try:  # torchrun exports OMP_NUM_THREADS=1: the CPU baseline is meant to use every host core it can
        torch.set_num_threads(max(1, len(os.sched_getaffinity(0))))
    except Exception:
        pass
    sample = min(args.batch, args.cpu_sample)
    base, sec = cpu_baseline_legs(args.batch, sample, max(1, args.steps))
    value = base["value"]
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": workload_config(args.batch),
        "cpu_baseline": base,
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


def run_reference_triton(args, rank, world):
    """`--impl reference-triton`: the reference's own Triton operator chain (partial_rope x2, paged_kv_append, split,
    combine, attention_gate_pack) for the same step on the GPU, replayed from a CUDA graph (rank 0 only)."""
    if rank != 0:
        return
    res, why = run_reference_task("op_bench", "triton", ["--steps", str(max(args.steps, 5)), "--batches", str(args.batch),
                                                         "--only", "decode_random"], 900)
    if res is None:
        emit({"impl": "reference-triton", "unavailable": why})
        return
    row = next(r for r in res["rows"] if r["op"] == "decode_chain" and r["B"] == args.batch and r["ctx"] == "random")
    nbytes = algorithmic_bytes(draw_lengths(args.batch, "random"))
    value = nbytes / (row["us"] * 1e-6) / 1e9
    emit({"impl": "reference-triton", "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
          "warmup": args.warmup, "ms_per_step": row["us"] * 1e-3, "higher_is_better": True, "scaling": "weak",
          "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": workload_config(args.batch),
          "gpu_launches": 6 * args.steps, "triton": res.get("triton"),
          "note": "the reference's six Triton launches per step, JIT-compiled by the installed Triton for this GPU"})


def claim_stdout():
    """stdout is for the one JSON line.  Libraries write there too (NCCL prints its version banner with printf), so the
    process's descriptor 1 is pointed at stderr for the whole run and the real stdout is kept aside for the result."""
    sys.stdout.flush()
    real = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    return real


RESULT_OUT = None


def emit(obj) -> None:
    out = RESULT_OUT if RESULT_OUT is not None else sys.stdout
    out.write(json.dumps(obj) + "\n")
    out.flush()


def main():
    global RESULT_OUT
    RESULT_OUT = claim_stdout()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference", "reference-triton"])
    ap.add_argument("--no-reference-triton", action="store_true",
                    help="skip the legs that run the reference's Triton kernels and runner on the GPU")
    ap.add_argument("--no-sweep", action="store_true")
    ap.add_argument("--cpu-sample", type=int, default=256)
    ap.add_argument("--sweep-steps", type=int, default=20)
    ap.add_argument("--kernel-only", action="store_true", help="headline timing only (for profiler captures)")
    ap.add_argument("--no-graph", action="store_true", help="launch every step from Python instead of one CUDA graph")
    ap.add_argument("--no-model", action="store_true", help="skip the whole-model decode measurement (24-layer random-init model)")
    ap.add_argument("--model-steps", type=int, default=512)
    ap.add_argument("--workload", default="decode", choices=["decode", "chain", "prefill", "gdn", "gdn_decode", "gemm", "model_prefill"],
                    help="with --kernel-only: which kernel family to run (profiler captures of the other families)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if args.impl == "reference-triton":
        run_reference_triton(args, rank, world)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path (use --impl reference for the CPU oracle)")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)

    from b200attn import ops

    if args.kernel_only and args.workload != "decode":
        if args.workload == "gemm":
            rows = run_gemm_sweep(ops, device, hbm_peak()[0], args.steps)
        elif args.workload == "gdn_decode":
            rows = run_gdn_decode_rows(ops, device, hbm_peak()[0], args.steps, (args.batch,))
        elif args.workload == "model_prefill":
            rows = run_model_prefill_rows(device, args.steps)
        elif args.workload == "chain":   # the drop-in operator chain (rope x2, append, split, combine, gate-pack)
            lengths = draw_lengths(args.batch, "random")
            w = Workload(lengths, device, max_sets=32)
            scratch = ops.allocate_split_scratch(HQ, D, batch=args.batch, device=device)
            ms = time_steps(chain_step(ops, w, scratch), args.steps, 3)
            rows = [{"op": "decode_chain", "B": args.batch, "us_per_layer": ms * 1e3, "gbs": w.bytes / (ms * 1e-3) / 1e9}]
        else:
            rows = run_prefill_sweep(ops, device, args.steps, only=args.workload)
        if rank == 0:
            emit({"kernel_only": True, "workload": args.workload, "rows": rows})
        if dist is not None:
            dist.destroy_process_group()
        return

    ws = ops.fused_decode_workspace(device)
    peak, peak_kind = hbm_peak()
    # weak scaling: every rank serves the same length distribution (BASELINE config 2, seed 1), so per-GPU work is fixed;
    # contents and page permutations differ per rank
    lengths = draw_lengths(args.batch, "random", seed=1)
    w = Workload(lengths, device, seed=1 + rank, pin_host=True)
    step = fused_step(ops, w, ws)

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()

    # ---- headline: device-resident inputs; the K timed steps are one CUDA-graph replay (as the engine decodes)
    for i in range(args.warmup):
        step(i)
    graph = None
    if not args.no_graph:
        graph = capture_steps(step, args.steps, args.warmup)
    barrier()
    with ClockSampler(local_rank) as clocks:
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        if graph is not None:
            graph.replay()
        else:
            for i in range(args.steps):
                step(args.warmup + i)
        end.record()
        barrier()
        ms_total = start.elapsed_time(end)
        # keep the sampler alive for a moment on very short runs so that it sees the load
        if ms_total < 400:
            t_end = time.time() + 0.5
            j = 0
            while time.time() < t_end:
                step(j)
                j += 1
            torch.cuda.synchronize()
    clock_info = clocks.summary()
    ms_total, total_bytes = aggregate_over_ranks(ms_total, float(w.bytes), dist, device)
    ms_per_step = ms_total / args.steps
    value = total_bytes / (ms_per_step * 1e-3) / 1e9

    if args.kernel_only:
        if rank == 0:
            emit({"metric": METRIC, "value": value, "unit": "GB/s", "ms_per_step": ms_per_step, "steps": args.steps,
                  "batch": args.batch, "kernel_only": True})
        if dist is not None:
            dist.destroy_process_group()
        return

    # ---- e2e: host inputs and output through the public operator
    e2e = e2e_step(ops, w, ws)
    for i in range(args.warmup):
        e2e(i)
    barrier()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    start.record()
    for i in range(args.steps):
        e2e(args.warmup + i)
    end.record()
    barrier()
    e2e_ms = max(start.elapsed_time(end), (time.perf_counter() - t0) * 1e3)
    e2e_ms, _ = aggregate_over_ranks(e2e_ms, 0.0, dist, device)
    e2e_value = total_bytes / (e2e_ms / args.steps * 1e-3) / 1e9
    h2d = args.batch * (4096 + 1024 + 1024 + 4096)
    d2h = args.batch * 4096

    line = {
        "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": workload_config(args.batch),
        "run": {"cache_sets": w.sets, "mb_per_step": w.bytes / 1e6,
                "launch": "python loop" if args.no_graph else "the K timed steps replayed from one CUDA graph",
                "parallelism": f"replicas x{world} (no data-path collective)", "us_per_layer": ms_per_step * 1e3},
        "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": e2e_ms / args.steps,
                "note": "public operator per step; pinned-host inputs in and result out every step, copies "
                        "double-buffered on side streams; wall clock around a device-wide synchronize"},
        "gpu_launches": args.steps,
        "clocks": clock_info,
    }

    if rank == 0:
        per_gpu = w.bytes / (ms_per_step * 1e-3) / 1e9
        line["roofline"] = {
            "bound": "hbm", "achieved": per_gpu, "peak": peak, "unit": "GB/s", "frac": per_gpu / peak,
            "traffic": (None if NCU_TRAFFIC_RATIO is None else NCU_TRAFFIC_RATIO * w.bytes),
            "traffic_source": "profiler capture of this launch shape, scaled by the algorithmic bytes",
            "peak_kind": f"of {peak_kind}", "kernel": "fused_decode_kernel",
            "algorithmic_bytes_per_launch": w.bytes,
        }
    sweep = None
    if world == 1 and not args.no_sweep:
        del step, e2e, graph
        sweep = run_sweep(ops, ws, device, peak, args.sweep_steps)
    if not args.no_model:
        del w
        torch.cuda.empty_cache()
        model = run_whole_model(device, rank, world, dist, args.model_steps, peak)
    else:
        model = None
    if world == 1:
        # ---- the reference beside it: its Triton kernels on this GPU, its CPU path on the host cores
        torch.cuda.empty_cache()
        if not args.no_reference_triton:
            line["reference_triton"] = reference_triton_legs(args, sweep, model, value)
        sample = min(args.batch, args.cpu_sample)
        line["cpu_baseline"], _ = cpu_baseline_legs(args.batch, sample, 3)
        if sweep is not None:
            line["sweep"] = sweep
    if model is not None and rank == 0:
        line["whole_model"] = model          # last: the end of the line survives truncated logs
    if rank == 0:
        emit(line)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def reference_triton_legs(args, sweep, model, value):
    """Runs the reference's Triton operator chains at the sweep's shapes and its runner on the whole-model workload (on
    its own kernels and on this package's drop-in operators) in child processes; writes `triton_us` into the matching
    sweep rows and returns the summary object."""
    out = {}
    batches = "1,4,16,32,64,256" if sweep is not None else str(args.batch)
    res, why = run_reference_task("op_bench", "triton", ["--steps", "10", "--batches", batches]
                                  + ([] if sweep is not None else ["--only", "decode_random"]), 900)
    if res is None:
        return {"unavailable": why}
    out["triton"] = res.get("triton")
    by_key = {}
    for r in res["rows"]:
        by_key[(r["op"], r.get("B"), r.get("ctx"), r.get("shape"))] = r["us"]
    head = by_key.get(("decode_chain", args.batch, "random", None))
    if head is not None:
        nbytes = algorithmic_bytes(draw_lengths(args.batch, "random"))
        out["headline_step"] = {"us_per_layer": head, "gbs": nbytes / (head * 1e-6) / 1e9,
                                "launches": 6, "speedup_of_fused_kernel": value / (nbytes / (head * 1e-6) / 1e9)}
    if sweep is not None:
        alias = {"fused_decode": "decode_chain", "fused_prefill_attention": "prefill_attention_layer_chain",
                 "gdn chunk-64 prefill, one sequence (drop-in entry point)": "gdn chunk-64 pipeline (3 launches)"}
        for row in sweep:
            op = alias.get(row["op"], row["op"])
            us = by_key.get((op, row.get("B"), row.get("ctx"), row.get("shape")))
            if us is None and op.startswith("gdn_chunked_prefill_fused"):
                us = by_key.get(("gdn_recurrent_prefill_sequential", None, None, row.get("shape")))   # its only packed route
            if us is not None:
                row["triton_us"] = us
        out["rows"] = res["rows"]
    if model is not None:
        extra = ["--batch", str(model["batch_per_gpu"]), "--prompt-len", str(model["prompt_len"]), "--steps",
                 str(min(model["decode_steps"], 256))]
        for kernels, key in (("triton", "runner_on_triton"), ("b200", "runner_on_dropin_operators"),
                             ("b200-fast", "fast_runner_subclass")):
            r, why = run_reference_task("model_bench", kernels, extra, 900)
            out[key] = {"unavailable": why} if r is None else {k: r[k] for k in ("ms_per_step", "tok_s", "prefill_ms",
                                                                                   "decode_steps", "batch")}
    return out


def run_model_prefill_rows(device, steps, batch=32, prompt_len=128):
    """The engine's packed prefill alone (random-init Qwen3.5-0.8B architecture, seed 4; 32 prompts x 128 random ids):
    `steps` calls after two untimed ones, each timed from the first host instruction to the last kernel."""
    from b200attn import engine as E
    cfg = E.ModelConfig()
    weights = E.random_weights(cfg, seed=4, device=device)
    gen = torch.Generator().manual_seed(4)
    prompts = [torch.randint(0, cfg.vocab, (prompt_len,), generator=gen).tolist() for _ in range(batch)]
    eng = E.Engine(cfg, weights, batch, prompt_len + 8, device, page_seed=0)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    times = []
    for i in range(steps + 2):
        eng.pos.zero_()
        torch.cuda.synchronize()
        start.record()
        eng.prefill(prompts)
        end.record()
        torch.cuda.synchronize()
        if i >= 2:
            times.append(start.elapsed_time(end))
    times.sort()
    return [{"op": "engine packed prefill", "shape": f"{batch}x{prompt_len}", "ms_median": times[len(times) // 2],
             "ms_min": times[0], "tok_s": batch * prompt_len / (times[len(times) // 2] * 1e-3)}]


def run_whole_model(device, rank, world, dist, steps, peak, batch=32, prompt_len=128, warm=4):
    """Whole-model workload: random-init Qwen3.5-0.8B architecture (seed 4), packed prefill of 32 prompts x 128 random
    token ids per GPU, then `steps` greedy decode steps replayed from one CUDA graph per step.  Attention and
    Gated-DeltaNet run on this package's kernels, the rest is PyTorch glue (cuBLAS GEMMs).  Every rank is an independent
    replica; with more than one rank the sampled ids are all-gathered over NCCL after every step (the only
    collective).  Reports whole-job tokens/s (max time over ranks) and the fraction of the HBM bound of one step:
    all weights once + Gated-DeltaNet states in and out + the KV cache of the mean context."""
    from b200attn import engine as E
    cfg = E.ModelConfig()
    weights = E.random_weights(cfg, seed=4, device=device)
    gen = torch.Generator().manual_seed(4 + rank)
    prompts = [torch.randint(0, cfg.vocab, (prompt_len,), generator=gen).tolist() for _ in range(batch)]
    eng = E.Engine(cfg, weights, batch, prompt_len + steps + warm + 2, device, page_seed=rank)

    def sync():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()

    eng.prefill(prompts)                       # first call: library handles, tensor maps, allocator pools
    eng.pos.zero_()
    sync()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    prefill_runs = []
    for _ in range(3):                         # host preparation and launches included; the median of three calls
        start.record()
        eng.prefill(prompts)
        end.record()
        sync()
        prefill_runs.append(start.elapsed_time(end))
        eng.pos.zero_()
        sync()
    eng.prefill(prompts)                       # the decode steps below continue from a filled cache
    sync()
    prefill_ms = sorted(prefill_runs)[1]
    for _ in range(warm):
        eng.step()
    eng.capture()
    # Multi-GPU: the sampled ids of every rank are gathered over NCCL, but not on the stream that decodes.  Each step
    # copies its ids into a small device history (one 256-byte copy between two graph replays); every GATHER_EVERY steps
    # a side stream all-gathers the filled half of the history while the compute stream goes on writing the other
    # half.  Events order "half filled -> gather" and "gather done -> half reused".
    GATHER_EVERY = 16
    if dist is not None:
        hist = torch.zeros(2, GATHER_EVERY, batch, dtype=torch.int64, device=device)
        gathered = torch.empty(world, GATHER_EVERY, batch, dtype=torch.int64, device=device)
        comm = torch.cuda.Stream(device=device)
        gather_done = [None, None]
    sync()
    start.record()
    for i in range(steps):
        tok = eng.step()
        if dist is not None:
            half, slot = (i // GATHER_EVERY) & 1, i % GATHER_EVERY
            if slot == 0 and gather_done[half] is not None:
                torch.cuda.current_stream(device).wait_event(gather_done[half])
            hist[half, slot].copy_(tok, non_blocking=True)
            if slot == GATHER_EVERY - 1 or i == steps - 1:
                filled = torch.cuda.Event()
                filled.record(torch.cuda.current_stream(device))
                with torch.cuda.stream(comm):
                    comm.wait_event(filled)
                    dist.all_gather_into_tensor(gathered.view(-1), hist[half].view(-1))
                    gather_done[half] = torch.cuda.Event()
                    gather_done[half].record(comm)
    if dist is not None:
        torch.cuda.current_stream(device).wait_stream(comm)   # the last gather is inside the timed region
    end.record()
    sync()
    ms = start.elapsed_time(end)
    if dist is not None:
        t = torch.tensor([ms, prefill_ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, prefill_ms = float(t[0]), float(t[1])
    param_bytes = sum(t.numel() * t.element_size() for t in [weights["embed"], weights["norm"]])
    for layer in weights["layers"]:
        param_bytes += sum(t.numel() * t.element_size() for k, t in layer.items()
                           if isinstance(t, torch.Tensor) and k != "conv")
    n_gdn = sum(1 for l in weights["layers"] if l["kind"] == "gdn")
    n_att = cfg.num_layers - n_gdn
    mean_ctx = prompt_len + warm + steps / 2
    step_bytes = param_bytes + n_gdn * batch * gdn_decode_bytes(1) + n_att * batch * 2048 * mean_ctx
    ms_step = ms / steps
    return {"metric": "whole-model greedy decode tokens/s (random-init Qwen3.5-0.8B architecture, bf16)",
            "value": world * batch * steps / (ms * 1e-3), "unit": "tok/s", "ms_per_step": ms_step,
            "batch_per_gpu": batch, "prompt_len": prompt_len, "decode_steps": steps, "n_gpus": world,
            "prefill_ms": prefill_ms, "prefill_tok_s": world * batch * prompt_len / (prefill_ms * 1e-3),
            "hbm_bytes_per_step_per_gpu": step_bytes, "hbm_frac": step_bytes / (ms_step * 1e-3) / 1e9 / peak,
            "launch": ("one CUDA graph per decode step; ids of 16 steps all-gathered over NCCL on a side stream"
                       if dist is not None else "one CUDA graph per decode step")}


def run_sweep(ops, ws, device, peak, steps):
    rows = []
    for mode in ("random", "fixed32768"):
        for b in (1, 4, 16, 32, 64, 256):
            lengths = draw_lengths(b, mode)
            w = Workload(lengths, device, max_sets=32)
            ms = time_steps(fused_step(ops, w, ws), steps, 3)
            row = {"op": "fused_decode", "B": b, "ctx": mode, "us_per_layer": ms * 1e3,
                   "gbs": w.bytes / (ms * 1e-3) / 1e9}
            row["frac"] = row["gbs"] / peak
            if mode == "random" or b <= 32:
                scratch = ops.allocate_split_scratch(HQ, D, batch=b, device=device)
                ms_c = time_steps(chain_step(ops, w, scratch), steps, 3)
                row["chain_us_per_layer"] = ms_c * 1e3
                row["chain_gbs"] = w.bytes / (ms_c * 1e-3) / 1e9
                # the same operator calls with the runner's decode symbol forced onto the reference's launch structure
                # (append -> split -> combine through the scratch tensors) instead of its one-launch form
                ops.DECODE_CALL_ONE_LAUNCH = False
                try:
                    ms_s = time_steps(chain_step(ops, w, scratch), steps, 3)
                finally:
                    ops.DECODE_CALL_ONE_LAUNCH = True
                row["chain_split_combine_us"] = ms_s * 1e3
                del scratch
            rows.append(row)
            del w
            torch.cuda.empty_cache()
    rows += run_gdn_decode_rows(ops, device, peak, steps, (1, 32, 256))
    rows += run_gemm_sweep(ops, device, peak, steps)
    rows += run_prefill_sweep(ops, device, steps)
    return rows


def run_gdn_decode_rows(ops, device, peak, steps, batches):
    """Gated-DeltaNet decode: fp32 state [B,16,128,128] streamed in and out once per step."""
    rows = []
    for b in batches:
        nbytes = gdn_decode_bytes(b)
        sets = max(1, min(32, cdiv(3 * L2_BYTES, nbytes)))
        states = [torch.zeros(b, 16, 128, 128, device=device) for _ in range(sets)]
        gen = torch.Generator().manual_seed(3)
        q = torch.nn.functional.normalize(torch.randn(b, 16, 128, generator=gen), dim=-1).to(torch.bfloat16).to(device)
        k = torch.nn.functional.normalize(torch.randn(b, 16, 128, generator=gen), dim=-1).to(torch.bfloat16).to(device)
        v = torch.randn(b, 16, 128, generator=gen).to(torch.bfloat16).to(device)
        beta = torch.sigmoid(torch.randn(b, 16, generator=gen)).to(device)
        g = (-torch.nn.functional.softplus(torch.randn(b, 16, generator=gen))).to(device)
        ms = time_steps(lambda i: ops.gdn_recurrent_decode(q, k, v, beta, g, states[i % sets]), steps, 3)
        rows.append({"op": "gdn_recurrent_decode", "B": b, "us_per_layer": ms * 1e3, "gbs": nbytes / (ms * 1e-3) / 1e9,
                     "frac": nbytes / (ms * 1e-3) / 1e9 / peak})
        # the whole mixer of a layer in one launch (conv + SiLU, norms, gates, the step above, gated RMSNorm): the same
        # state bytes plus the conv state [B, 4, 6144] bf16 in and out
        kd = 16 * 128
        w4 = (torch.randn(4, 3 * kd, generator=gen) * 0.5).to(torch.bfloat16).to(device)
        a_log = (torch.rand(16, generator=gen) * 2.7).to(device)
        dt_bias = (torch.randn(16, generator=gen) * 0.5).to(torch.bfloat16).to(device)
        norm_w = (1 + 0.1 * torch.randn(128, generator=gen)).to(device)
        convs = [torch.zeros(b, 4, 3 * kd, dtype=torch.bfloat16, device=device) for _ in range(sets)]
        row_in = torch.randn(b, 4 * kd + 32, generator=gen).to(torch.bfloat16).to(device)
        ms = time_steps(lambda i: ops.gdn_decode_fused(row_in, convs[i % sets], w4, a_log, dt_bias, norm_w,
                                                       states[i % sets], 16), steps, 3)
        mbytes = nbytes + 2 * b * 4 * 3 * kd * 2
        rows.append({"op": "gdn_decode_fused (mixer, one launch)", "B": b, "us_per_layer": ms * 1e3,
                     "gbs": mbytes / (ms * 1e-3) / 1e9, "frac": mbytes / (ms * 1e-3) / 1e9 / peak})
        del states, convs
        torch.cuda.empty_cache()
    return rows


def run_gemm_sweep(ops, device, peak, steps):
    """The decode-step projections of the whole-model workload (32 sequences, hidden 1024): weight-streaming GEMMs, bound by the
    weight bytes.  Weights rotate over enough copies that no call finds its matrix in L2; the cuBLAS time of the same
    product (plus torch.argmax for the LM head) is reported beside each."""
    import torch.nn.functional as F
    rows = []
    gen = torch.Generator().manual_seed(5)
    m = 32
    shapes = (("input projection (GDN layer)", 8224, 1024, "plain"), ("gate/up projection + SwiGLU", 7168, 1024, "swiglu"),
              ("output projection", 1024, 2048, "plain"), ("down projection", 1024, 3584, "plain"),
              ("LM head + arg-max", 248320, 1024, "argmax"))
    ws_arg = ops.argmax_workspace(device)
    for tag, n, k, kind in shapes:
        nbytes = n * k * 2
        copies = max(2, min(48, cdiv(3 * L2_BYTES, nbytes)))
        x = torch.randn(m, k, generator=gen).to(torch.bfloat16).to(device)
        weights = [(torch.randn(n, k, device=device) * 0.03).to(torch.bfloat16) for _ in range(copies)]
        if kind == "swiglu":
            own = lambda i: ops.skinny_gemm(x, weights[i % copies], swiglu=True)
            lib = lambda i: ops.swiglu_fused(F.linear(x, weights[i % copies]), n // 2)
        elif kind == "argmax":
            own = lambda i: ops.lm_head_argmax(x, weights[i % copies], ws_arg)
            lib = lambda i: torch.argmax(torch.mm(x, weights[i % copies].t(), out_dtype=torch.float32), dim=-1)
        else:
            own = lambda i: ops.skinny_gemm(x, weights[i % copies])
            lib = lambda i: F.linear(x, weights[i % copies])
        ms = time_steps(own, steps, 3)
        ms_lib = time_steps(lib, steps, 3)
        rows.append({"op": "decode GEMM: " + tag, "shape": f"[{m},{k}] x [{n},{k}]^T", "us": ms * 1e3,
                     "gbs": nbytes / (ms * 1e-3) / 1e9, "frac_hbm": nbytes / (ms * 1e-3) / 1e9 / peak,
                     "cublas_us": ms_lib * 1e3})
        del weights
        torch.cuda.empty_cache()
    return rows


def run_prefill_sweep(ops, device, steps, only=None):
    """Prefill-side operators at the benchmark shapes: packed varlen causal attention (B=32, lengths
    ~U[16,512] seed 2, plus a long-prompt shape where the tensor bound applies) and the GDN prefill forms (config 4:
    32 prompts x 128 tokens).  Reported against both rooflines; inputs are regenerated per call site, not rotated
    (every call reads each input once, outputs are larger than the reuse L2 could give)."""
    rows = []
    tf_peak = 1649.6
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            tf_peak = float(json.loads(p.read_text())["bf16_tflops"])
        except Exception:
            pass
    hbm, _ = hbm_peak()
    gen = torch.Generator().manual_seed(2)
    attn_shapes = (("cfg3 B=32 L~U[16,512]", torch.randint(16, 513, (32,), generator=gen).tolist()),
                   ("long B=8 L=4096", [4096] * 8))
    if only == "prefill":
        attn_shapes = attn_shapes[1:]
    elif only == "gdn":
        attn_shapes = ()
    for tag, lengths in attn_shapes:
        total = sum(lengths)
        q = torch.randn(total, HQ, D, device=device, dtype=torch.bfloat16)
        k = torch.randn(total, HKV, D, device=device, dtype=torch.bfloat16)
        v = torch.randn(total, HKV, D, device=device, dtype=torch.bfloat16)
        gate = torch.randn(total, HQ * D, device=device, dtype=torch.bfloat16)
        cu, max_len = ops.build_cu_seqlens(lengths, device=device)
        flops = 4096 * sum(n * (n + 1) for n in lengths)
        nbytes = total * (4096 + 1024 + 1024 + 4096)
        ms = time_steps(lambda i: ops.gqa_attention_varlen_causal(q, k, v, cu, max_len), steps, 3)
        rows.append({"op": "gqa_attention_varlen_causal", "shape": tag, "tokens": total, "us": ms * 1e3,
                     "tflops": flops / (ms * 1e-3) / 1e12, "frac_tensor": flops / (ms * 1e-3) / 1e12 / tf_peak,
                     "gbs": nbytes / (ms * 1e-3) / 1e9, "frac_hbm": nbytes / (ms * 1e-3) / 1e9 / hbm})
        pps = [cdiv(n, PAGE) for n in lengths]
        table = torch.zeros(len(lengths), max(pps), dtype=torch.int32)
        perm = torch.randperm(sum(pps), generator=gen)
        off = 0
        for i, n in enumerate(pps):
            table[i, :n] = perm[off:off + n].to(torch.int32)
            off += n
        table = table.to(device)
        kc, vc = ops.allocate_paged_kv_cache(sum(pps), HKV, D, device=device)
        ids = torch.cat([torch.arange(n) for n in lengths]).to(torch.int32).to(device)
        inv = (1.0 / (1e7 ** (torch.arange(0, ROT, 2, dtype=torch.float32) / ROT))).to(device)
        out = torch.empty(total, HQ * D, dtype=torch.bfloat16, device=device)
        ms = time_steps(lambda i: ops.fused_prefill_attention(q, k, v, gate, kc, vc, table, cu, ids, inv, ROT, max_len,
                                                              out=out), steps, 3)
        nbytes_f = nbytes + total * (4096 + 2048)
        rows.append({"op": "fused_prefill_attention", "shape": tag, "tokens": total, "us": ms * 1e3,
                     "tflops": flops / (ms * 1e-3) / 1e12, "frac_tensor": flops / (ms * 1e-3) / 1e12 / tf_peak,
                     "gbs": nbytes_f / (ms * 1e-3) / 1e9, "frac_hbm": nbytes_f / (ms * 1e-3) / 1e9 / hbm})
        del q, k, v, gate, kc, vc, out
        torch.cuda.empty_cache()
    if only == "prefill":
        return rows
    # GDN prefill, config 4: 32 prompts x 128 tokens, 16 heads
    heads, lengths = 16, [128] * 32
    total = sum(lengths)
    gq = torch.nn.functional.normalize(torch.randn(total, heads, 128, generator=gen), dim=-1) * 128 ** -0.5
    gk = torch.nn.functional.normalize(torch.randn(total, heads, 128, generator=gen), dim=-1)
    gq, gk = gq.to(torch.bfloat16).to(device), gk.to(torch.bfloat16).to(device)
    gv = torch.randn(total, heads, 128, generator=gen).to(torch.bfloat16).to(device)
    beta = torch.sigmoid(torch.randn(total, heads, generator=gen)).to(device)
    g = (-torch.nn.functional.softplus(torch.randn(total, heads, generator=gen))
         * torch.exp(torch.rand(heads, generator=gen) * 2.7)).to(device)
    cu, _ = ops.build_cu_seqlens(lengths, device=device)
    flops = total * heads * 7 * 128 * 128  # seven 128x128 fp32 multiply-adds-ish per token per head
    nbytes = total * heads * 128 * 2 * 4 + len(lengths) * heads * 128 * 128 * 4
    ms = time_steps(lambda i: _gdn_seq_nosync(ops, gq, gk, gv, beta, g, cu, len(lengths)), steps, 3)
    rows.append({"op": "gdn_recurrent_prefill_sequential", "shape": "cfg4 B=32 x 128", "tokens": total, "us": ms * 1e3,
                 "tflops_fp32": flops / (ms * 1e-3) / 1e12, "gbs": nbytes / (ms * 1e-3) / 1e9})
    # chunk-64 on the tensor cores: 12.1 MFLOP per (chunk, head) counting each product once; bytes = q, k, v read,
    # out written (bf16), beta and g read, final state written
    ms = time_steps(lambda i: ops.gdn_chunked_prefill_packed(gq, gk, gv, beta, g, cu), steps, 3)
    cflops = 12.1e6 * 2 * len(lengths) * heads
    cbytes = total * heads * (4 * 128 * 2 + 8) + len(lengths) * heads * 128 * 128 * 4
    rows.append({"op": "gdn_chunked_prefill_fused (tcgen05, 1 launch)", "shape": "cfg4 B=32 x 128", "tokens": total,
                 "us": ms * 1e3, "tflops": cflops / (ms * 1e-3) / 1e12, "frac_tensor": cflops / (ms * 1e-3) / 1e12 / tf_peak,
                 "gbs": cbytes / (ms * 1e-3) / 1e9, "frac_hbm": cbytes / (ms * 1e-3) / 1e9 / hbm})
    ms = time_steps(lambda i: ops.gdn_chunked_prefill_packed(gq, gk, gv, beta, g, cu, 128, fused=False), steps, 3)
    rows.append({"op": "gdn_chunked_prefill_packed (3 launches)", "shape": "cfg4 B=32 x 128", "tokens": total,
                 "us": ms * 1e3, "tflops": cflops / (ms * 1e-3) / 1e12, "frac_tensor": cflops / (ms * 1e-3) / 1e12 / tf_peak})
    # the same kernel where every SM has work for many chunks: 32 prompts x 1024 tokens (512 CTAs x 16 chunks)
    long_len = [1024] * 32
    lt = sum(long_len)
    gen2 = torch.Generator().manual_seed(11)
    lq = torch.nn.functional.normalize(torch.randn(lt, heads, 128, generator=gen2), dim=-1) * 128 ** -0.5
    lk = torch.nn.functional.normalize(torch.randn(lt, heads, 128, generator=gen2), dim=-1)
    lq, lk = lq.to(torch.bfloat16).to(device), lk.to(torch.bfloat16).to(device)
    lv = torch.randn(lt, heads, 128, generator=gen2).to(torch.bfloat16).to(device)
    lbeta = torch.sigmoid(torch.randn(lt, heads, generator=gen2)).to(device)
    lg = (-torch.nn.functional.softplus(torch.randn(lt, heads, generator=gen2))
          * torch.exp(torch.rand(heads, generator=gen2) * 2.7)).to(device)
    lcu, _ = ops.build_cu_seqlens(long_len, device=device)
    ms = time_steps(lambda i: ops.gdn_chunked_prefill_packed(lq, lk, lv, lbeta, lg, lcu), steps, 3)
    lflops = 12.1e6 * (lt // 64) * heads
    lbytes = lt * heads * (4 * 128 * 2 + 8) + len(long_len) * heads * 128 * 128 * 4
    rows.append({"op": "gdn_chunked_prefill_fused (tcgen05, 1 launch)", "shape": "B=32 x 1024", "tokens": lt,
                 "us": ms * 1e3, "tflops": lflops / (ms * 1e-3) / 1e12, "frac_tensor": lflops / (ms * 1e-3) / 1e12 / tf_peak,
                 "gbs": lbytes / (ms * 1e-3) / 1e9, "frac_hbm": lbytes / (ms * 1e-3) / 1e9 / hbm})
    del lq, lk, lv, lbeta, lg
    # one sequence through the drop-in entry point the reference runner calls for long prompts (engine/runner.py:272-273)
    for n_tok in (128, 2048):
        gen1 = torch.Generator().manual_seed(3)
        sq = (torch.nn.functional.normalize(torch.randn(n_tok, heads, 128, generator=gen1), dim=-1) * 128 ** -0.5)
        sk = torch.nn.functional.normalize(torch.randn(n_tok, heads, 128, generator=gen1), dim=-1)
        sq, sk = sq.to(torch.bfloat16).to(device), sk.to(torch.bfloat16).to(device)
        sv = torch.randn(n_tok, heads, 128, generator=gen1).to(torch.bfloat16).to(device)
        sb = torch.sigmoid(torch.randn(n_tok, heads, generator=gen1)).to(device)
        sg = (-torch.nn.functional.softplus(torch.randn(n_tok, heads, generator=gen1))
              * torch.exp(torch.rand(heads, generator=gen1) * 2.7)).to(device)
        ms = time_steps(lambda i: ops.call_gdn_recurrent_prefill_chunked_triton(sq, sk, sv, sb, sg), steps, 3)
        rows.append({"op": "gdn chunk-64 prefill, one sequence (drop-in entry point)", "shape": f"1 x {n_tok}",
                     "tokens": n_tok, "us": ms * 1e3})
    return rows


def _gdn_seq_nosync(ops, q, k, v, beta, g, cu, batch):
    """gdn_recurrent_prefill_sequential through the C ABI without the operator's host read of cu_seqlens[-1] (the
    reference's assert), so that it can sit inside a CUDA graph."""
    from b200attn import _lib
    total, heads, dk = q.shape
    out = torch.empty_like(v)
    state = torch.empty(batch, heads, dk, v.shape[-1], dtype=torch.float32, device=q.device)
    _lib.call("b200_gdn_recurrent_prefill_sequential", q.data_ptr(), q.stride(0), q.stride(1), k.data_ptr(), k.stride(0),
              k.stride(1), v.data_ptr(), v.stride(0), v.stride(1), beta.data_ptr(), beta.stride(0), beta.stride(1),
              g.data_ptr(), g.stride(0), g.stride(1), cu.data_ptr(), batch, total, state.data_ptr(), out.data_ptr(),
              out.stride(0), out.stride(1), heads, dk, v.shape[-1], torch.cuda.current_stream().cuda_stream)
    return out


if __name__ == "__main__":
    main()
