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


def _expert_parallel_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    sys.path.insert(0, ROOT)
    from oracle import moe_oracle as MO
    T, H, k, e_local, cap = 96, 64, 4, 4, 1024
    g = torch.Generator().manual_seed(100 + rank)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    ids, _ = MO.route(torch.randn(T, world * e_local, generator=g), k)
    ids_all = [torch.empty_like(ids) for _ in range(world)]
    x_all = [torch.empty_like(x) for _ in range(world)]
    dist.all_gather(ids_all, ids)
    dist.all_gather(x_all, x)
    # every rank derives its own schedule from the gathered routing decisions, with no further exchange
    pr, pt, nt, tpe, written = MO.schedule_ref(torch.stack(ids_all), e_local, cap, rank)
    n = int(nt)
    valid = torch.tensor([int((pr[:n] >= 0).sum())])
    dist.all_reduce(valid)
    # identity experts: what a rank's experts return is what dispatch brought them
    y = torch.zeros(cap, H, dtype=torch.bfloat16)
    y[:n] = MO.dispatch_ref(torch.stack(x_all), pr, pt, n, k)
    meta = torch.full((2, cap), -1, dtype=torch.int32)
    meta[0, :n], meta[1, :n] = pr[:n], pt[:n]
    ys = [torch.empty_like(y) for _ in range(world)]
    metas = [torch.empty_like(meta) for _ in range(world)]
    dist.all_gather(ys, y)
    dist.all_gather(metas, meta)
    buf = MO.combine_ref(ys, [m[0] for m in metas], [m[1] for m in metas], rank, T, k)
    # each (token, slot) pair was served by exactly one expert somewhere: its combine row holds the token again
    whole = torch.equal(buf.view(T, k, H).view(torch.int16), x.view(T, 1, H).expand(T, k, H).contiguous().view(torch.int16))
    q.put((rank, int(valid.item()), whole, int(tpe.sum()) == n and n % 256 == 0))
    dist.barrier()
    dist.destroy_process_group()


def test_expert_parallel_exchange_covers_every_routed_pair_once_gloo():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_expert_parallel_worker, args=(r, 2, 29543, q)) for r in range(2)]
    for p in procs:
        p.start()
    out = sorted(q.get(timeout=180) for _ in procs)
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    assert [o[1] for o in out] == [2 * 96 * 4] * 2          # valid rows over both ranks = world * tokens * top-k
    assert all(o[2] and o[3] for o in out)
