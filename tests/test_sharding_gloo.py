"""The multi-GPU harness logic of bench.py on CPU: world_size-2 gloo ranks take disjoint batch
shards, no collective touches the data path, and the reported time is the maximum over ranks."""
import os
import sys

import torch as th
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    import bench
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port))
    dist.init_process_group('gloo', rank=rank, world_size=world)
    lo, hi = bench.shard_of(rank, world, 7)
    slowest = bench.max_over_ranks(10.0 + rank, dist, th.device('cpu'))
    covered = th.zeros(7)
    covered[lo:hi] = 1
    dist.all_reduce(covered)  # harness-side check only
    if rank == 0:
        out.put((slowest, covered.tolist()))
    dist.destroy_process_group()


def test_two_ranks_cover_the_batch_once_and_report_the_slowest_rank():
    ctx = mp.get_context('spawn')
    out = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    slowest, covered = out.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert slowest == 11.0
    assert covered == [1.0] * 7


def test_shard_of_partitions_exactly():
    import bench
    for total in (1, 7, 64, 65):
        for world in (1, 2, 4, 8):
            spans = [bench.shard_of(r, world, total) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
