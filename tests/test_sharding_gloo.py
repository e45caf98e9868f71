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


# ---- the (batch x kv-head) shard partition ----

def test_every_shard_is_assigned_exactly_once():
    from adasplash_b200 import sharding as sh
    for B, Hkv, lens in ((2, 8, None), (4, 32, None), (8, 8, [16384, 5000, 9000, 4096, 12000, 16000, 7000, 4100])):
        shards = sh.enumerate_shards(B, Hkv, 16384, lens)
        assert [s.shard_id for s in shards] == list(range(B * Hkv))
        for world in (1, 2, 3, 4, 8):
            parts = sh.assign(shards, world)
            assert len(parts) == world
            ids = sorted(s.shard_id for part in parts for s in part)
            assert ids == list(range(B * Hkv))


def test_equal_lengths_split_evenly_round_robin():
    from adasplash_b200 import sharding as sh
    shards = sh.enumerate_shards(2, 8, 65536)          # the long-context configuration: 16 shards
    for world, per in ((1, 16), (2, 8), (4, 4), (8, 2)):
        parts = sh.assign(shards, world)
        assert [len(p) for p in parts] == [per] * world
        assert [s.shard_id for s in parts[0]] == list(range(0, 16, world))


def test_varlen_balance_bound():
    from adasplash_b200 import sharding as sh
    g = torch.Generator().manual_seed(11)
    for trial in range(20):
        B, Hkv, N = 8, 8, 16384
        lens = [int(x) for x in torch.randint(N // 4, N + 1, (B,), generator=g)]
        shards = sh.enumerate_shards(B, Hkv, N, lens)
        for world in (2, 4, 8):
            load = sh.loads(sh.assign(shards, world))
            mean = sum(load) / world
            heaviest = max(s.weight for s in shards)
            assert max(load) <= mean + heaviest            # longest-processing-time bound
            assert max(load) <= 4 / 3 * mean + heaviest / 3 + 1


def _shard_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from adasplash_b200 import sharding as sh
    lens = [64, 40]
    shards = sh.enumerate_shards(2, 2, 64, lens)
    mine = sh.assign(shards, world)[rank]
    batch = sh.make_rank_batch(mine, G=2, N=64, D=16, seed=20264, scale=1.5, dtype=torch.float32)
    q, k, v, do, varlen = batch
    out[rank] = {s.shard_id: (q[i].clone(), k[i].clone(), do[i].clone(), s.length) for i, s in enumerate(mine)}
    out[("varlen", rank)] = None if varlen is None else varlen.tolist()
    dist.barrier()
    dist.destroy_process_group()


def test_shard_tensors_identical_at_world_1_and_2():
    from adasplash_b200 import sharding as sh
    shards = sh.enumerate_shards(2, 2, 64, [64, 40])
    one = sh.make_rank_batch(sh.assign(shards, 1)[0], G=2, N=64, D=16, seed=20264, scale=1.5, dtype=torch.float32)
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_shard_worker, args=(2, 29633, out), nprocs=2, join=True)
        res = dict(out)
    seen = {}
    for r in range(2):
        seen.update(res[r])
    assert sorted(seen) == [0, 1, 2, 3]
    for sid, (q, k, do, L) in seen.items():
        assert torch.equal(q, one[0][sid]) and torch.equal(k, one[1][sid]) and torch.equal(do, one[3][sid])
        assert do[:, L:].abs().sum() == 0                  # dO is zero beyond the shard's length
    # lengths [64, 40] x 2 kv heads by weight: rank 0 gets a long and a short shard, and so does rank 1
    assert sorted(res[("varlen", 0)]) == [40, 64] and sorted(res[("varlen", 1)]) == [40, 64]
