"""Host-side logic of the multi-GPU benchmark, run with two gloo ranks on CPU: shard arithmetic,
the max-over-ranks reduction, and the reference arm that only rank 0 runs."""
import json
import os
import subprocess
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    sys.path.insert(0, ROOT)
    import bench
    # rows of A and C split across ranks, B replicated: shards tile the matrix exactly
    M, rows = bench.gemm_shard_rows(world)
    lo = rank * rows
    cover = torch.zeros(M, dtype=torch.int32)
    cover[lo:lo + rows] = 1
    dist.all_reduce(cover)
    # the slowest rank defines the step time
    t = torch.tensor([10.0 + rank], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    q.put((rank, rows, bool((cover == 1).all()), float(t.item())))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_sharding_gloo():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, 29541, q)) for r in range(2)]
    for p in procs:
        p.start()
    out = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    assert [o[1] for o in out] == [4096, 4096]
    assert all(o[2] for o in out)
    assert all(o[3] == 11.0 for o in out)


def test_shard_rows_every_world_size():
    sys.path.insert(0, ROOT)
    import bench
    for n in (1, 2, 4, 8):
        M, rows = bench.gemm_shard_rows(n)
        assert rows * n == M == 8192 and rows % 128 == 0


def test_reference_arm_runs_on_rank0_only():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1"],
                       capture_output=True, text=True, env=env, timeout=300)
    assert r.returncode == 0 and r.stdout.strip() == ""
    env = dict(os.environ, RANK="0", WORLD_SIZE="2")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1",
                        "--warmup", "3"], capture_output=True, text=True, env=env, timeout=300)
    assert r.returncode == 0
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["cpu_baseline"]["kind"] == "port" and line["value"] > 0
    assert line["e2e"]["h2d_bytes_per_step"] == 0
