"""Host-side logic of the benchmark: site order, and the multi-rank aggregation run as two
gloo ranks on CPU (the data path itself has no collective)."""
import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import bench


def test_site_order_matches_engine_layout():
    o = bench.site_order(bench.LOCAL)
    assert len(o) == 42 and o[:3] == [0, 1, 2] and o[-3:] == [9, 10, 11]
    assert o[3:9] == [3, 4, 5, 6, 7, 8] and o[9:15] == [3, 4, 5, 6, 7, 8]
    assert len(bench.site_order(bench.CLOUD)) == 72
    assert bench.job_throughput(64 * 10, 8, 1000.0) == 64 * 10 * 8


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        slow = bench.max_over_ranks(10.0 * (rank + 1), torch.device("cpu"))
        out[rank] = (slow, bench.job_throughput(640, world, slow))
    finally:
        dist.destroy_process_group()


def test_two_rank_aggregation_uses_slowest_rank():
    world = 2
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_worker, args=(world, 29511 + os.getpid() % 200, out), nprocs=world, join=True)
        res = dict(out)
    assert res[0][0] == res[1][0] == 20.0
    assert res[0][1] == 640 * 2 / 0.020
