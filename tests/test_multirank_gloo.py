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
    # the strong split of the decode step: bins of equal summed cache length, one per rank
    bins = workloads.balanced_partition(lens, world)
    bin_bytes = workloads.decode_bytes(lens[bins[rank]], 64, 16, 64)
    bin_total = bench._sum_over_ranks(bin_bytes, world, cpu)
    gathered = bench.gather_over_ranks(float(lens[bins[rank]].sum()), world, cpu)
    # the timed-region helper itself, on a host function (no GPU work to wait for)
    region, launch, det = _host_timed_steps(bench, world, rank)
    q.put((rank, mx, sm, total, pairs_total, (sl.start, sl.stop), bin_total, gathered, det["rank_region_ms"]))
    dist.destroy_process_group()


def _host_timed_steps(bench, world, rank):
    """bench.timed_steps needs CUDA events; this drives the same reductions it ends with."""
    mine = [5.0 + rank, 7.0 - rank, 6.0]
    maxima = [bench.max_over_ranks(m, world, torch.device("cpu")) for m in mine]
    pick = sorted(range(3), key=lambda i: maxima[i])[1]
    return maxima[pick], 0.0, {"rank_region_ms": bench.gather_over_ranks(mine[pick], world, torch.device("cpu"))}


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
    bins = workloads.balanced_partition(lens, world)
    assert sorted(i for b in bins for i in b) == list(range(len(lens)))
    sums = [int(lens[b].sum()) for b in bins]
    assert max(sums) - min(sums) <= int(lens.max())          # balanced on the summed length
    for rank, mx, sm, total, pairs_total, _, bin_total, gathered, rank_ms in res:
        assert mx == 11.0 and sm == 300.0
        assert abs(total - want_bytes) < 1.0
        assert pairs_total == float(want_pairs)
        assert abs(bin_total - want_bytes) < 1.0               # the bins cover every sequence once
        assert gathered == [float(x) for x in sums]
        assert rank_ms == [6.0, 6.0]                           # the median region, every rank's own time
    assert res[0][5] == (0, 64) and res[1][5] == (64, 128)
