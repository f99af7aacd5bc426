"""Multi-GPU host logic on the CPU with two gloo ranks: streams are partitioned without overlap, ranks
exchange nothing on the data path, and the reported time is the maximum over ranks."""
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


def _worker(rank, world, port, streams_per_rank, out):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import bench
    seeds = list(range(rank * streams_per_rank, (rank + 1) * streams_per_rank))
    # every rank builds only its own streams (seed = global stream index)
    frames = bench.make_streams(streams_per_rank, first_seed=rank * streams_per_rank)
    assert frames.shape[1] == streams_per_rank
    checksum = torch.tensor([float(frames[:2].sum())])
    gathered = [torch.zeros(1) for _ in range(world)]
    dist.all_gather(gathered, checksum)
    # time reduction as in bench.py: max over ranks
    ms = torch.tensor([10.0 + 5.0 * rank])
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    out[rank] = (seeds, [float(g) for g in gathered], float(ms))
    dist.barrier()
    dist.destroy_process_group()


def test_stream_partition_and_time_reduction_two_ranks():
    world, per_rank = 2, 2
    port = _free_port()
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(world, port, per_rank, out), nprocs=world, join=True)
    seeds0, sums0, ms0 = out[0]
    seeds1, sums1, ms1 = out[1]
    assert set(seeds0).isdisjoint(seeds1) and sorted(seeds0 + seeds1) == [0, 1, 2, 3]
    assert sums0 == sums1 and sums0[0] != sums0[1]          # different streams on different ranks
    assert ms0 == ms1 == 15.0                              # max over ranks


def test_pingpong_indexing():
    sys.path.insert(0, ROOT)
    import bench
    n = 5
    idx = [bench.pingpong(t, n) for t in range(12)]
    assert idx == [0, 1, 2, 3, 4, 3, 2, 1, 0, 1, 2, 3]
    assert all(abs(a - b) == 1 for a, b in zip(idx, idx[1:]))   # consecutive frames are neighbours in time
