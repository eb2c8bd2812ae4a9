"""The N > 1 path of bench.py on CPU: two gloo ranks stand in for two GPUs. Replicas share nothing on
the data path; what they exchange is the timing reduction (MAX) and the job totals (SUM)."""
import json
import os
import subprocess
import sys
from pathlib import Path

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
import bench  # noqa: E402


def _rank(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    # Rank r "measured" r + 1 ms on the device and emitted 100 (r + 1) tokens with 10 launches.
    vals, sums = bench.reduce_over_ranks(dev_ms=1.0 + rank, wall_s=0.5 - 0.1 * rank, emitted=100 * (rank + 1), launches=10, world=world, device="cpu")
    dist.barrier()
    Path(out_dir, f"r{rank}.json").write_text(json.dumps({"vals": vals, "sums": sums}))
    dist.destroy_process_group()


def test_two_ranks_reduce_to_the_slowest_time_and_the_job_totals(tmp_path):
    port = 29500 + os.getpid() % 2000
    mp.spawn(_rank, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        got = json.loads((tmp_path / f"r{r}.json").read_text())
        assert got["vals"] == [2.0, 0.5]      # max over ranks of device ms and of wall seconds
        assert got["sums"] == [300.0, 20.0]   # whole-job tokens and launches


def test_streams_are_distinct_across_replicas():
    seeds = {bench.stream_seeds(r, j) for r in range(8) for j in range(32)}
    assert len(seeds) == 8 * 32
    assert len({s[0] for s in seeds}) == 8 * 32 and len({s[1] for s in seeds}) == 8 * 32
    assert bench.stream_seeds(0, 3)[0] == 10  # the reference's 7 + j on the first replica


def test_reference_arm_runs_on_rank_zero_only():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    r = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--gpus", "2"], env=env, capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and r.stdout.strip() == ""
