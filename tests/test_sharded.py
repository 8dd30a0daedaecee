"""Batch sharding over ranks: partition arithmetic, and the compute + all-gather path run as
two gloo ranks on CPU (the compute step is a stand-in that fills each item with its global
index; the GPU kernels are covered by the gpu tests)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from flextensor_b200.sharded import BatchSharded, chunk_ranges, shard_range


def test_shard_range_covers_the_batch_exactly():
    for batch in (1, 7, 64, 65):
        for world in (1, 2, 3, 4, 8):
            pieces = [shard_range(batch, world, r) for r in range(world)]
            assert pieces[0][0] == 0 and pieces[-1][1] == batch
            assert all(pieces[i][1] == pieces[i + 1][0] for i in range(world - 1))
            sizes = [hi - lo for lo, hi in pieces]
            assert max(sizes) - min(sizes) <= 1
    assert [shard_range(64, 8, r) for r in (0, 7)] == [(0, 8), (56, 64)]
    with pytest.raises(ValueError):
        shard_range(8, 2, 2)


def test_chunk_ranges():
    assert chunk_ranges(8, 1) == [(0, 8)]
    assert chunk_ranges(8, 3) == [(0, 3), (3, 6), (6, 8)]
    assert chunk_ranges(2, 5) == [(0, 1), (1, 2)]
    assert chunk_ranges(0, 2) == [(0, 0)]


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, batch, fail_rank, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        sh = BatchSharded(batch)
        out_local = torch.zeros(sh.local, 3, 5)
        out_full = torch.zeros(batch, 3, 5)

        def compute(lo, hi):
            if rank == fail_rank:
                raise RuntimeError("rank %d fails on the host" % rank)
            for i in range(lo, hi):
                out_local[i] = float(sh.lo + i)

        sh.run(compute, out_local, out_full, chunks=2)
        want = torch.arange(batch, dtype=torch.float32).view(batch, 1, 1).expand(batch, 3, 5)
        results[rank] = bool(torch.equal(out_full, want)) and (sh.lo, sh.hi) == shard_range(batch, world, rank)
    except Exception as exc:
        results[rank] = "error: %s" % exc
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


def _run(world, batch, fail_rank=-1):
    ctx = mp.get_context("spawn")
    results = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, batch, fail_rank, results)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        if p.is_alive():
            p.terminate()
    return dict(results)


def test_two_ranks_compute_and_gather():
    results = _run(2, 8)
    assert results == {0: True, 1: True}


def test_uneven_batch_is_refused():
    results = _run(2, 7)
    assert all(isinstance(v, str) and "multiple of the world size" in v for v in results.values())
