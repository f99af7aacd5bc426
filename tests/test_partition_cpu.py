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


def _checksum_worker(rank, world, port, total, out):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import bench
    ids = bench.stream_ids(rank, world, 0, total)
    outputs = torch.stack([_fake_logits(s) for s in ids])          # what this rank's streams produced
    sums = bench.stream_checksums(outputs)
    gathered = [None] * world
    dist.all_gather_object(gathered, (ids, sums))
    all_ids = [i for part in gathered for i in part[0]]
    all_sums = [v for part in gathered for v in part[1]]
    out[rank] = (ids, bench.combine_checksums(all_ids, all_sums))
    dist.barrier()
    dist.destroy_process_group()


def _fake_logits(stream_id):
    g = torch.Generator().manual_seed(1000 + stream_id)
    return torch.randn(10, generator=g)


def test_round_robin_partition_gives_the_one_gpu_checksum():
    """Streams dealt round-robin to two ranks (stream s on rank s mod 2): the digest over all streams' outputs equals
    the digest of a single process running every stream, and changes when any stream's output changes."""
    sys.path.insert(0, ROOT)
    import bench
    world, total = 2, 6
    port = _free_port()
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_checksum_worker, args=(world, port, total, out), nprocs=world, join=True)
    assert out[0][0] == [0, 2, 4] and out[1][0] == [1, 3, 5]
    single_ids = bench.stream_ids(0, 1, 0, total)
    single = bench.combine_checksums(single_ids, bench.stream_checksums(torch.stack([_fake_logits(s) for s in single_ids])))
    assert out[0][1] == out[1][1] == single
    changed = [_fake_logits(s) for s in single_ids]
    changed[3] = changed[3] + 1e-6
    assert bench.combine_checksums(single_ids, bench.stream_checksums(torch.stack(changed))) != single
    assert bench.stream_ids(1, 4, 16) == list(range(16, 32))
