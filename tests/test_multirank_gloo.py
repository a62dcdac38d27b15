"""The N > 1 path on CPU: two gloo ranks run the benchmark's sharding and reduction helpers
(shards disjoint and complete, timing = max over ranks, work = sum over ranks)."""

import os
import socket
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank),
                      WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    import bench
    from sps_b200 import workloads
    dist.init_process_group("gloo", rank=rank, world_size=world)
    cpu = torch.device("cpu")
    mx = bench.max_over_ranks(10.0 + rank, world, cpu)
    sm = bench._sum_over_ranks(100.0 * (rank + 1), world, cpu)
    bench.barrier(world)
    # this rank's shard of the decode sequences and its share of the algorithmic bytes
    lens = workloads.decode_lengths("cfg2_segmented_decode")
    sl = workloads.shard_slice(len(lens), rank, world)
    mine = workloads.decode_bytes(lens[sl], 64, 16, 64)
    total = bench._sum_over_ranks(mine, world, cpu)
    docs = workloads.geometric_docs(8, 512, 100, 0)
    pairs = workloads.useful_pairs(docs[workloads.shard_slice(8, rank, world)], 64)
    pairs_total = bench._sum_over_ranks(float(pairs), world, cpu)
    q.put((rank, mx, sm, total, pairs_total, (sl.start, sl.stop)))
    dist.destroy_process_group()


def test_two_gloo_ranks_shard_and_reduce():
    from sps_b200 import workloads
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    lens = workloads.decode_lengths("cfg2_segmented_decode")
    want_bytes = workloads.decode_bytes(lens, 64, 16, 64)
    want_pairs = workloads.useful_pairs(workloads.geometric_docs(8, 512, 100, 0), 64)
    for rank, mx, sm, total, pairs_total, _ in res:
        assert mx == 11.0 and sm == 300.0
        assert abs(total - want_bytes) < 1.0
        assert pairs_total == float(want_pairs)
    assert res[0][5] == (0, 64) and res[1][5] == (64, 128)
