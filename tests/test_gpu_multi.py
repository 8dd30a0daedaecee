"""Two or more GPUs: batch-sharded batched GEMM, conv2d and depthwise conv2d, the output returned
to every rank by the kernels themselves (stores into every rank's buffer over NVLink), by
device-to-device pushes, and by an NCCL all-gather - each rank checking the whole gathered result
against the oracle.  Skipped on a single-GPU box.

Ranks are child processes, one per GPU.  NVLS is switched off for NCCL and symmetric memory is
told not to bind a multicast object (``TORCH_SYMM_MEM_DISABLE_MULTICAST=1``); the kernels use
plain peer stores.  The ranks agree on the host (a gloo all-reduce of a flag) that every launch
went through before any of them enters a device-side barrier, so a rank whose launch failed
cannot leave its peers waiting; every rank drops its symmetric buffers and destroys the process
group on every exit path, and a rank only leaves between steps, with nothing in flight.
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
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0",
                      TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    import torch.distributed as dist
    from flextensor_b200 import backend as B
    from flextensor_b200.sharded import BatchSharded, PeerGatheredOutput, ShardedOp, shard_range
    from flextensor_b200.task import batch_gemm, conv2d, depthwise_conv2d
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    host = dist.new_group(backend="gloo")       # host-side agreement, never touches a GPU
    outcome = {}
    opened = []

    def all_ranks_ok(local_ok):
        flag = torch.tensor([1 if local_ok else 0], dtype=torch.int32)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=host)
        return bool(flag.item())

    def dev(x):
        return torch.from_numpy(np.ascontiguousarray(x)).to(device)

    def run_sharded(name, op, inputs, check):
        """launch -> agree on the host -> device barrier / gather -> compare the gathered output"""
        opened.append(op)
        err = None
        try:
            op.launch(*inputs)
            torch.cuda.synchronize()
        except Exception as exc:  # recorded; the peers learn of it before they wait for this rank
            err = "%s: %s" % (type(exc).__name__, exc)
        if not all_ranks_ok(err is None):
            outcome[name] = err or "a peer's launch failed"
            return
        op.finish()
        torch.cuda.synchronize()
        op.check()
        outcome[name] = bool(check(op.out_full))
        if op.gather == "fused":
            outcome[name + "_by_kernel"] = bool(op.func.pushed_by_kernel)

    try:
        # ---- batched GEMM bf16: raw multi-destination entry point, then the same through the task interface
        batch, m, n, k = 2 * world, 256, 384, 192
        lo, hi = shard_range(batch, world, rank)
        items = [O.batch_gemm_item(i, m, n, k, seed=71) for i in range(batch)]
        want = O.batch_gemm(np.stack([i[0] for i in items]), np.stack([i[1] for i in items]))
        a = dev(np.stack([i[0] for i in items[lo:hi]])).bfloat16()
        b = dev(np.stack([i[1] for i in items[lo:hi]])).bfloat16()
        status = B.new_status(device)
        out = PeerGatheredOutput(batch, m, n, dtype=torch.bfloat16)
        out.tensor.fill_(float("nan"))
        dist.barrier()
        err = None
        try:
            B.bgemm_bf16_multi(a, b, out.slice_ptrs(lo), m, n, status=status)
            torch.cuda.synchronize()
        except Exception as exc:
            err = "%s: %s" % (type(exc).__name__, exc)
        if all_ranks_ok(err is None):
            out.barrier()
            torch.cuda.synchronize()
            outcome["bgemm_raw_fused"] = bool(O.bf16_output_ok(out.tensor.float().cpu().numpy(), want))
        else:
            outcome["bgemm_raw_fused"] = err or "a peer's launch failed"
        fused_copy = out.tensor.clone()
        out.close()
        sh = BatchSharded(batch)
        c_local = torch.empty(hi - lo, m, n, device=device, dtype=torch.bfloat16)
        c_full = torch.full((batch, m, n), float("nan"), device=device, dtype=torch.bfloat16)
        sh.run(lambda l, h: B.bgemm_bf16(a[l:h], b[l:h], c_local[l:h], status=status), c_local, c_full, chunks=2)
        torch.cuda.synchronize()
        outcome["bgemm_nccl"] = bool(O.bf16_output_ok(c_full.float().cpu().numpy(), want)) and \
            bool(torch.equal(c_full, fused_copy))
        B.check_status(status)
        for mode in ("fused", "nccl"):
            op = ShardedOp("gemm", "batch_gemm", batch_gemm, (batch, m, k, n), gather=mode)
            run_sharded("bgemm_module_" + mode, op, (a, b),
                        lambda full: O.bf16_output_ok(full.float().cpu().numpy(), want))
        # ---- conv2d (grouped, 3 channels per group) and depthwise conv2d, images sharded over the ranks
        nimg = 2 * world
        x, w = O.conv2d_inputs(nimg, 12, 14, 16, 24, 3, 3, groups=4, seed=72)
        want_conv = O.conv2d_nchw(x, w, None, 1, 1, 1, 4)
        lo, hi = shard_range(nimg, world, rank)
        for mode in ("fused", "push", "nccl"):
            op = ShardedOp("conv2d", "sharded", conv2d, (nimg, 12, 14, 16, 24, 3, 1, 1, 1, 4), gather=mode)
            run_sharded("conv2d_" + mode, op, (dev(x[lo:hi]), dev(w)),
                        lambda full: O.normalised_error(full.cpu().numpy(), want_conv) <= O.TOLERANCE["conv2d_tf32"])
        # one group, stride 1: the slab kernel, whose epilogue also stores into every rank's buffer
        xs, ws_ = O.conv2d_inputs(nimg, 32, 14, 16, 40, 3, 3, seed=74)
        want_slab = O.conv2d_nchw(xs, ws_, None, 1, 1, 1, 1)
        op = ShardedOp("conv2d", "sharded_slab", conv2d, (nimg, 32, 14, 16, 40, 3, 1, 1, 1, 1), gather="fused")
        run_sharded("conv2d_slab_fused", op, (dev(xs[lo:hi]), dev(ws_)),
                    lambda full: O.normalised_error(full.cpu().numpy(), want_slab) <= O.TOLERANCE["conv2d_tf32"])
        # output rows of 15 floats cannot leave through bulk stores: one destination, pushed afterwards
        xo, wo = O.conv2d_inputs(nimg, 8, 9, 15, 8, 3, 3, seed=75)
        want_odd = O.conv2d_nchw(xo, wo, None, 1, 1, 1, 1)
        op = ShardedOp("conv2d", "sharded_odd", conv2d, (nimg, 8, 9, 15, 8, 3, 1, 1, 1, 1), gather="fused")
        run_sharded("conv2d_odd_fused", op, (dev(xo[lo:hi]), dev(wo)),
                    lambda full: O.normalised_error(full.cpu().numpy(), want_odd) <= O.TOLERANCE["conv2d_tf32"])
        xd, wd = O.depthwise_inputs(nimg, 16, 28, 28, 2, 3, 3, seed=73)
        want_dw = O.depthwise_conv2d_nchw(xd, wd, None, 1, 1, 1)
        for mode in ("fused", "push", "nccl"):
            op = ShardedOp("conv2d", "depthwise", depthwise_conv2d, (nimg, 16, 28, 28, 2, 3, 1, 1, 1), gather=mode)
            run_sharded("depthwise_" + mode, op, (dev(xd[lo:hi]), dev(wd)),
                        lambda full: O.normalised_error(full.cpu().numpy(), want_dw) <= O.TOLERANCE["depthwise_f32"])
        results[rank] = dict(outcome)
    except Exception as exc:
        outcome["error"] = "%s: %s" % (type(exc).__name__, exc)
        results[rank] = dict(outcome)
    finally:
        try:
            torch.cuda.synchronize()
        except Exception:
            pass
        for op in opened:
            op.close()
        try:
            dist.destroy_process_group()
        except Exception:
            pass


EXPECTED = {"bgemm_raw_fused": True, "bgemm_nccl": True, "bgemm_module_fused": True, "bgemm_module_fused_by_kernel": True,
            "bgemm_module_nccl": True, "conv2d_fused": True, "conv2d_fused_by_kernel": True, "conv2d_push": True,
            "conv2d_nccl": True, "conv2d_slab_fused": True, "conv2d_slab_fused_by_kernel": True,
            "conv2d_odd_fused": True, "conv2d_odd_fused_by_kernel": False,
            "depthwise_fused": True, "depthwise_fused_by_kernel": True, "depthwise_push": True,
            "depthwise_nccl": True}


def test_sharded_operators_fused_push_and_nccl(native_lib):
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
        p.join(timeout=600)
    stuck = [p for p in procs if p.is_alive()]
    for p in stuck:
        p.terminate()
    assert not stuck, "ranks did not finish"
    assert dict(results) == {r: EXPECTED for r in range(world)}


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
