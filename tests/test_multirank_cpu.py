"""The N > 1 plumbing of bench.py on CPU ranks (gloo, world_size 2): every rank takes its own shard of the batch (the
scan has no data-path collective), the step time is the MAX over ranks and throughput counts all ranks' tokens."""
import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import bench
    inp = bench.make_host_inputs(2, 16, 3, 16, 16, seed=rank)            # each rank: its own sequences
    ms, ms2 = bench.max_over_ranks([10.0 + rank, 5.0 - rank], "cpu")     # rank 1 is slower on the first, faster on the second
    q.put((rank, float(inp["k"].sum()), ms, ms2))
    dist.destroy_process_group()


def test_two_gloo_ranks_shard_and_reduce():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    ps = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in ps:
        p.start()
    out = sorted(q.get(timeout=120) for _ in ps)
    for p in ps:
        p.join(timeout=60)
        assert p.exitcode == 0
    (r0, s0, a0, b0), (r1, s1, a1, b1) = out
    assert s0 != s1                          # different shards of the batch
    assert a0 == a1 == 11.0 and b0 == b1 == 5.0      # max over ranks, identical on every rank
    import bench
    assert bench.whole_job_tokens_per_s(64, 1024, 2, 10, 50.0) == 2 * 64 * 1024 * 10 / 0.05


def test_strong_scaling_shards_cover_the_global_batch():
    import bench
    for world in (1, 2, 4, 8, 3):
        parts = [bench.shard_of_batch(64, world, r, "strong") for r in range(world)]
        assert sum(n for _, n in parts) == 64
        assert [f for f, _ in parts] == [sum(n for _, n in parts[:r]) for r in range(world)]     # contiguous, in rank order
        assert max(n for _, n in parts) - min(n for _, n in parts) <= 1
    assert bench.shard_of_batch(64, 8, 3, "strong") == (24, 8)
    assert bench.shard_of_batch(64, 8, 3, "weak") == (192, 64)
    # CPU sample of the reference arm: at least two OpenMP tasks per host thread
    for cores in (8, 16, 32, 64):
        assert bench.cpu_sample_batch(cores, 6) * 6 >= 2 * cores
