"""The N>1 host logic of the bench on CPU ranks (gloo, world_size 2): sharding of independent images, max-over-ranks of
the per-rank device time, whole-job rate.  No collective exists on the data path, so this is all there is to test."""
import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import bench
    dist.init_process_group("gloo", rank=rank, world_size=world)
    my_ms = 10.0 + 5.0 * rank                      # rank 1 is the slow one
    ms = bench.max_over_ranks(my_ms, world, "cpu")
    plan = bench.shard_plan(513, world)
    dist.barrier()
    out.put((rank, ms, plan, bench.whole_job_rate(plan, 4, ms)))
    dist.destroy_process_group()


def test_two_ranks_agree_on_the_slowest_time_and_the_job_rate():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, 29731, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, ms, plan, rate in res:
        assert ms == 15.0                                   # max over ranks, on every rank
        assert plan == [257, 256] and sum(plan) == 513      # remainder to the low ranks
        assert abs(rate - 513 * 4 / 0.015) < 1e-6


def test_shard_plan_edges():
    import bench
    assert bench.shard_plan(1, 8) == [1, 0, 0, 0, 0, 0, 0, 0]    # batch 1: replicas only, one rank works
    assert bench.shard_plan(256, 8) == [32] * 8
    assert bench.shard_plan(0, 2) == [0, 0]
