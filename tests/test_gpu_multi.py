"""Two or more GPUs: the batch-sharded batched GEMM with the gather fused into the epilogue
(bulk stores into every rank's output over NVLink) and with the NCCL all-gather, each rank
checking the whole gathered result against the oracle.  Skipped on a single-GPU box.

Ranks are child processes, one per GPU; NVLS is switched off for NCCL and the kernels use plain
peer stores, so a rank that fails cannot leave a multicast binding behind.  A rank only leaves
between steps, with nothing in flight.
"""
import os
import socket

import numpy as np
import pytest
import torch

from oracle import ft_oracle as O

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _rank_main(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    from flextensor_b200 import backend as B
    from flextensor_b200.sharded import BatchSharded, PeerGatheredOutput, shard_range
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    try:
        batch, m, n, k = 2 * world, 256, 384, 192
        lo, hi = shard_range(batch, world, rank)
        items = [O.batch_gemm_item(i, m, n, k, seed=71) for i in range(batch)]
        want = O.batch_gemm(np.stack([i[0] for i in items]), np.stack([i[1] for i in items]))
        a = torch.from_numpy(np.stack([i[0] for i in items[lo:hi]])).to(device).bfloat16()
        b = torch.from_numpy(np.stack([i[1] for i in items[lo:hi]])).to(device).bfloat16()
        status = B.new_status(device)
        # fused: epilogue stores into every rank's buffer, then one barrier
        out = PeerGatheredOutput(batch, m, n, torch.bfloat16)
        out.tensor.fill_(float("nan"))
        dist.barrier()
        B.bgemm_bf16_multi(a, b, out.slice_ptrs(lo), m, n, status=status)
        out.barrier()
        torch.cuda.synchronize()
        fused_ok = O.bf16_output_ok(out.tensor.float().cpu().numpy(), want)
        # NCCL: local compute, all-gather
        sh = BatchSharded(batch)
        c_local = torch.empty(hi - lo, m, n, device=device, dtype=torch.bfloat16)
        c_full = torch.full((batch, m, n), float("nan"), device=device, dtype=torch.bfloat16)
        sh.run(lambda l, h: B.bgemm_bf16(a[l:h], b[l:h], c_local[l:h], status=status), c_local, c_full, chunks=2)
        torch.cuda.synchronize()
        nccl_ok = O.bf16_output_ok(c_full.float().cpu().numpy(), want)
        B.check_status(status)
        results[rank] = (bool(fused_ok), bool(nccl_ok), bool(torch.equal(c_full, out.tensor)))
        dist.barrier()
    except Exception as exc:
        results[rank] = "error: %s: %s" % (type(exc).__name__, exc)
    finally:
        dist.destroy_process_group()


def test_sharded_bgemm_fused_and_nccl(native_lib):
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    results = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, results)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
        if p.is_alive():
            p.terminate()
    assert dict(results) == {r: (True, True, True) for r in range(world)}


def test_measurement_pool_uses_every_gpu(native_lib):
    """Candidates are measured one per GPU in parallel worker processes."""
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least two GPUs")
    from flextensor_b200.measure import GpuPoolMeasurer
    from flextensor_b200.task import TASK_TABLE
    from flextensor_b200.templates import knobs_to_config
    from flextensor_b200.utils import Config
    key = "gemm_batch_gemm_(4, 256, 512, 384)_cuda(0)"
    op = TASK_TABLE[key].func(*TASK_TABLE[key].args)[0][0]
    jobs = []
    for i in range(3 * n):
        cluster = 1 + i % 2                       # a pair stages half of tile_n per CTA: at least one 64-wide box
        knobs = {"tile_n": (128, 256)[i % 2] if cluster == 2 else (64, 128, 256)[i % 3], "cluster": cluster,
                 "stages": 2 + i % 3}
        jobs.append((key, Config([knobs_to_config(knobs, op)], None), None))
    pool = GpuPoolMeasurer(devices=list(range(n)))
    try:
        results = pool(jobs, number=3, timeout=60, parallel=n)
        serial = pool(jobs[:2], number=3, timeout=60, parallel=1)
    finally:
        pool.close()
    assert all(0 < r < 100 for r in results), results
    assert all(0 < r < 100 for r in serial)
    assert {dev for _, _, _, dev in pool.trace[:len(jobs)]} == set(range(n))
    assert {dev for _, _, _, dev in pool.trace[len(jobs):]} == {0}
