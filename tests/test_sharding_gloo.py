"""Multi-GPU logic of the benchmark on CPU: two gloo ranks.

The (batch x kv-head) shards are independent, so a multi-GPU run has no
collective on the data path; what the ranks share is the per-rank seeding of
the inputs and the max-over-ranks reduction of the elapsed time.  Both are
checked here with world_size = 2 on the gloo backend (no GPU involved).
"""
import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

TINY = dict(B=2, Hq=4, Hkv=2, N=64, D=16, scale=1.5, varlen=True, label="tiny")


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import bench
    q, k, v, do, varlen, lens = bench.make_inputs(TINY, rank, pinned=False)
    # the slowest rank defines the step time
    ms = bench.max_over_ranks(10.0 + 5.0 * rank, world, torch.device("cpu"))
    flops = bench.dense_equiv_flops(TINY, lens)
    # ranks see different data; a rank failure elsewhere must not be needed to notice it
    sums = [torch.zeros(1) for _ in range(world)]
    dist.all_gather(sums, q.float().sum().reshape(1))
    out[rank] = dict(ms=ms, flops=flops, lens=lens, qsum=[float(x) for x in sums],
                     padded_do=float(do[0, :, lens[0]:].abs().sum()) if lens[0] < TINY["N"] else 0.0)
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_timing_and_seeding():
    world = 2
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_worker, args=(world, 29631, out), nprocs=world, join=True)
        res = dict(out)
    assert res[0]["ms"] == res[1]["ms"] == 15.0           # max over ranks
    assert res[0]["qsum"] == res[1]["qsum"]                # both saw the same gathered values
    assert res[0]["qsum"][0] != res[0]["qsum"][1]          # per-rank seeds give different shards
    for r in range(world):
        assert all(TINY["N"] // 4 <= l <= TINY["N"] for l in res[r]["lens"])
        assert res[r]["padded_do"] == 0.0                  # dO is zero on padded rows
        assert res[r]["flops"] == 7.0 * TINY["Hq"] * TINY["D"] * sum(l * l for l in res[r]["lens"])


def test_aggregate_is_whole_job_throughput():
    import bench
    one = bench.aggregate_tflops(1, 7.7e12, 25.0)
    assert abs(one - 308.0) < 1e-9
    assert abs(bench.aggregate_tflops(8, 7.7e12, 25.0) - 8 * one) < 1e-9


def test_inputs_are_deterministic_per_rank():
    import bench
    a = bench.make_inputs(TINY, 3, pinned=False)
    b = bench.make_inputs(TINY, 3, pinned=False)
    assert all(torch.equal(x, y) for x, y in zip(a[:4], b[:4])) and a[5] == b[5]
