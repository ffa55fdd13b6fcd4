"""Host-side logic of the multi-GPU path on CPU: chunk sharding covers the batch exactly once,
and a world_size-2 gloo job reproduces the max-over-ranks timing reduction that bench.py uses
(no collective touches the data path)."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from fluke_b200.shard import shard_chunks, shard_range


def test_shard_ranges_partition_the_batch():
    for n in (0, 1, 7, 128, 1024, 1025):
        for world in (1, 2, 3, 4, 8):
            spans = [shard_range(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            sizes = [e - b for b, e in spans]
            assert max(sizes) - min(sizes) <= 1


def test_shard_chunks_is_a_view_of_the_right_rows():
    x = torch.arange(5 * 10 * 3).view(5, 10, 3)
    parts = [shard_chunks(x, r, 4, 1) for r in range(4)]
    assert torch.equal(torch.cat(parts, dim=1), x)


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from bench import reduce_step_time, local_units
    units = local_units(1024, 1000, 5)             # weak scaling: every rank owns a full batch
    ms = reduce_step_time(10.0 + 5.0 * rank)       # max over ranks
    tot = torch.tensor([units], dtype=torch.float64)
    dist.all_reduce(tot)
    if rank == 0:
        out.put((ms, tot.item()))
    dist.destroy_process_group()


def test_gloo_world2_timing_reduction():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    [p.start() for p in procs]
    ms, tot = q.get(timeout=120)
    [p.join(60) for p in procs]
    assert ms == 15.0 and tot == 2 * 1024 * 1000 * 5


def test_strong_scaling_record_and_roofline_fractions():
    """The strong-scaling sub-record of the bench line (1024 chunks in total over the ranks) and
    the fractions quoted for the GEMM entries."""
    from bench import roofline_fractions, strong_scaling_record
    r = strong_scaling_record(1024, 8, 10.0)
    assert r["chunks_per_gpu"] == 128 and r["chunks_total"] == 1024
    assert r["value"] == 1024 * 1000 * 5 / 10e-3
    assert strong_scaling_record(1024, 3, 10.0)["chunks_per_gpu"] == 342   # the largest shard sets the time
    # 134.22 GOP and 149.7 MB in 50 us against 4500 TOP/s and 6538.6 GB/s: tensor floor 29.8 us, HBM floor 22.9 us
    ft, fh, ff = roofline_fractions(50.0, 134.22e9, 149.7e6, 4500.0, 6538.6)
    assert abs(ft - 0.597) < 2e-3 and abs(fh - 0.458) < 2e-3 and ff == ft
    ft, fh, ff = roofline_fractions(30.0, 50.33e9, 115.87e6, 4500.0, 6538.6)      # HBM-bound shape
    assert ff == fh and ft < fh
    assert roofline_fractions(10.0, 0.0, 65.79e6, None, 6538.6)[0] is None
