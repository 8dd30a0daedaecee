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


# ---------------------------------------------------------------- batch-sharded conv2d / depthwise (two gloo ranks)
def _conv_worker(rank, world, port, kind, results):
    """Each rank plans the Task of its images, runs a stand-in for the built module (the numpy
    oracle on the rank's slice; the CUDA kernels are covered by the gpu tests) and all-gathers."""
    import numpy as np
    from oracle import ft_oracle as O
    from flextensor_b200.sharded import ShardedOp
    from flextensor_b200.task import conv2d, depthwise_conv2d
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        batch = 6
        if kind == "conv2d":
            args = (batch, 8, 7, 9, 12, 3, 1, 1, 1, 2)           # N, C, H, W, K, kernel, stride, pad, dilation, groups
            x, w = O.conv2d_inputs(batch, 8, 7, 9, 12, 3, 3, groups=2, seed=90)
            want = O.conv2d_nchw(x, w, None, 1, 1, 1, 2)
            op = ShardedOp("conv2d", "sharded_test", conv2d, args, gather="nccl")
            stand_in = lambda xs, ws, out: out.copy_(torch.from_numpy(O.conv2d_nchw(xs.numpy(), ws.numpy(), None, 1, 1, 1, 2)))
        else:
            args = (batch, 5, 8, 8, 2, 3, 2, 1, 1)               # N, C, H, W, factor, kernel, stride, pad, dilation
            x, w = O.depthwise_inputs(batch, 5, 8, 8, 2, 3, 3, seed=91)
            want = O.depthwise_conv2d_nchw(x, w, None, 2, 1, 1)
            op = ShardedOp("conv2d", "depthwise_sharded_test", depthwise_conv2d, args, gather="nccl")
            stand_in = lambda xs, ws, out: out.copy_(torch.from_numpy(
                O.depthwise_conv2d_nchw(xs.numpy(), ws.numpy(), None, 2, 1, 1)))
        assert (op.lo, op.hi) == shard_range(batch, world, rank) and op.task.args[0] == batch // world
        assert tuple(op.bufs[0].shape)[0] == batch // world       # the rank's Task is planned on its slice
        assert tuple(op.out_full.shape) == want.shape
        op.func = stand_in
        got = op(torch.from_numpy(x[op.lo:op.hi]), torch.from_numpy(w))
        results[rank] = bool(np.allclose(got.numpy(), want, rtol=1e-5, atol=1e-6))
    except Exception as exc:
        results[rank] = "error: %s: %s" % (type(exc).__name__, exc)
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


@pytest.mark.parametrize("kind", ["conv2d", "depthwise_conv2d"])
def test_two_ranks_shard_a_conv_along_the_batch(kind):
    ctx = mp.get_context("spawn")
    results = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_conv_worker, args=(r, 2, port, kind, results)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=180)
        if p.is_alive():
            p.terminate()
    assert dict(results) == {0: True, 1: True}


def test_peer_gathered_output_disables_symmetric_memory_multicast(monkeypatch):
    """Only plain peer pointers are used, so the NVLink multicast binding is switched off before
    any rendezvous can happen - also when the constructor then fails (no process group here)."""
    import flextensor_b200.sharded as S
    monkeypatch.delenv(S.SYMM_MEM_ENV, raising=False)
    with pytest.raises(RuntimeError):
        S.PeerGatheredOutput(4, 8, 8, dtype=torch.float32)
    assert os.environ.get(S.SYMM_MEM_ENV) == "1"
