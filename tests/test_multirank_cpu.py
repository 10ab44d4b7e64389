"""The N > 1 host logic on CPU (gloo, world size 2): replicas only - each rank draws its own workload, the job time is
the slowest rank's, units add up, and only rank 0 reports; the sampled ids are all-gathered as the whole-model loop
does.  No GPU and no CUDA library call is involved."""
import json
import os
import socket
import subprocess
import sys
from pathlib import Path

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, result_dir: str):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    sys.path.insert(0, str(ROOT))
    import bench
    lengths = bench.draw_lengths(8, "random", seed=1 + rank)             # per-rank shard of the request batch
    ms, units = bench.aggregate_over_ranks(10.0 * (rank + 1), 100.0 + rank, dist, torch.device("cpu"))
    tok = torch.arange(4, dtype=torch.int64) + 10 * rank                  # this rank's sampled ids
    gathered = torch.empty(world * 4, dtype=torch.int64)
    dist.all_gather_into_tensor(gathered, tok)
    Path(result_dir, f"rank{rank}.json").write_text(json.dumps(
        {"ms": ms, "units": units, "lengths": lengths, "gathered": gathered.tolist()}))
    dist.barrier()
    dist.destroy_process_group()


def test_replica_aggregation_gloo(tmp_path):
    world, port = 2, _free_port()
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    r = [json.loads((tmp_path / f"rank{i}.json").read_text()) for i in range(world)]
    for x in r:
        assert x["ms"] == 20.0            # max over ranks
        assert x["units"] == 201.0        # sum over ranks
        assert x["gathered"] == [0, 1, 2, 3, 10, 11, 12, 13]
    assert r[0]["lengths"] != r[1]["lengths"]                             # every replica has its own sequences


def test_reference_arm_under_torchrun():
    """bench.py --impl reference launched as the driver launches it for N = 2: rank 0 alone runs the CPU oracle and
    prints the one JSON line, rank 1 exits 0 without work."""
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", str(_free_port()), str(ROOT / "bench.py"), "--impl", "reference", "--gpus", "2",
           "--steps", "1", "--warmup", "0", "--batch", "2", "--cpu-sample", "2"]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [json.loads(l) for l in res.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    line = lines[0]
    assert line["impl"] == "reference" and line["n_gpus"] == 2
    # the reference's own CPU code when its copy (baseline/_ref) is present, the oracle port otherwise
    assert line["cpu_baseline"]["kind"] in ("reference", "port") and line["cpu_baseline"]["value"] > 0
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["value"] > 0
