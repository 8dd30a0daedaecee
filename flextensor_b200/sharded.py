"""Batch-sharded execution over several GPUs of one node.

The reference runs every operator on one device (its only multi-device notion is the
``dev_id`` a task is pinned to, flextensor/task.py:226).  Batched GEMM, conv2d and depthwise
conv2d shard naturally along the batch axis: items are independent, so each rank computes its
contiguous slice with the single-GPU kernels, weights replicated, no data-path exchange; what
remains is returning the full output to every rank.  Three ways are built:

``fused``  The gathered output lives in symmetric memory (``PeerGatheredOutput``: every rank maps
           every rank's buffer over NVLink) and the kernel itself writes its slice into all
           ranks' buffers: the batched-GEMM epilogue with one bulk tensor store per slab and
           destination (``ftb_bgemm_bf16_multi``), the depthwise kernels with plain stores
           (``ftb_dwconv2d_nchw_f32_multi``).  The transfer overlaps the math; one barrier
           after the kernel is all that is left of the collective.
``push``   The kernel writes its slice into this rank's buffer only and device-to-device copies
           place it in the peers' buffers (conv2d, whose kernels have one destination).
``nccl``   The kernel writes a local slice; one ``all_gather_into_tensor`` follows
           (``BatchSharded``; ``run`` can overlap the gather of chunk i with the compute of
           chunk i+1).

The fused and push forms only ever *store* into peer memory through plain mapped pointers; no
load, and no library kernel, reads a peer's memory.  ``TORCH_SYMM_MEM_DISABLE_MULTICAST=1`` is
set before the symmetric-memory rendezvous so that no NVLink multicast object is bound to the
buffer: nothing here would use it, and a rank that dies while bound to one disturbs its peers.

One process per GPU; ``torch.distributed`` must be initialised by the caller.
"""
import os

import torch
import torch.distributed as dist

SYMM_MEM_ENV = "TORCH_SYMM_MEM_DISABLE_MULTICAST"


def disable_symm_mem_multicast():
    """Plain peer mappings only: must run before the first symmetric-memory rendezvous."""
    os.environ[SYMM_MEM_ENV] = "1"


disable_symm_mem_multicast()


def shard_range(batch, world_size, rank):
    """Contiguous slice [lo, hi) of ``batch`` items owned by ``rank``; the first
    ``batch % world_size`` ranks get one extra item."""
    if world_size < 1 or not (0 <= rank < world_size):
        raise ValueError("bad rank %d of %d" % (rank, world_size))
    base, extra = divmod(batch, world_size)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def chunk_ranges(count, chunks):
    """Split ``count`` local items into at most ``chunks`` contiguous, near-equal ranges."""
    chunks = max(1, min(chunks, count)) if count > 0 else 1
    out, lo = [], 0
    for i in range(chunks):
        hi = lo + count // chunks + (1 if i < count % chunks else 0)
        out.append((lo, hi))
        lo = hi
    return out


class BatchSharded(object):
    """Runs ``compute(lo, hi)`` over this rank's slice and all-gathers the output.

    compute : callable(lo, hi) launching the kernels for local items [lo, hi) into
              ``out_local[lo:hi]`` on the current stream
    out_local : this rank's output slice, shape [local_batch, ...]
    out_full  : the gathered output, shape [batch, ...]; requires batch % world_size == 0
                (equal slices, as ``all_gather`` needs)
    """

    def __init__(self, batch, group=None):
        if not dist.is_initialized():
            raise RuntimeError("torch.distributed is not initialised")
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if batch % self.world:
            raise ValueError("batch %d is not a multiple of the world size %d" % (batch, self.world))
        self.batch = batch
        self.lo, self.hi = shard_range(batch, self.world, self.rank)
        self.local = self.hi - self.lo
        self._comm_stream = None

    def gather(self, out_local, out_full):
        """One all-gather of the whole local slice (blocking on the current stream)."""
        if self.world == 1:
            if out_full.data_ptr() != out_local.data_ptr():
                out_full.copy_(out_local)
            return
        dist.all_gather_into_tensor(out_full, out_local, group=self.group)

    def run(self, compute, out_local, out_full, chunks=1):
        """compute + gather; with ``chunks > 1`` the gather of a chunk overlaps the next chunk's
        compute (CUDA tensors only)."""
        if chunks <= 1 or self.world == 1 or not out_local.is_cuda:
            compute(0, self.local)
            self.gather(out_local, out_full)
            return
        main = torch.cuda.current_stream()
        if self._comm_stream is None:
            self._comm_stream = torch.cuda.Stream(device=out_local.device)
        comm = self._comm_stream
        full_view = out_full.view(self.world, self.local, *out_full.shape[1:])
        for lo, hi in chunk_ranges(self.local, chunks):
            compute(lo, hi)
            done = torch.cuda.Event()
            done.record(main)
            comm.wait_event(done)
            with torch.cuda.stream(comm):
                # rank r's items [lo, hi) land at out_full[r*local + lo : r*local + hi]
                outs = [full_view[r, lo:hi] for r in range(self.world)]
                dist.all_gather(outs, out_local[lo:hi], group=self.group)
        main.wait_stream(comm)


class PeerSlice(object):
    """Items [lo, hi) of a ``PeerGatheredOutput`` as the *output argument* of a built module:
    ``func(*inputs, peer_out.slice(lo, hi))`` makes the kernel place its result in every rank's
    buffer (``runtime.Module.__call__`` recognises it).  ``tensor`` is the local view,
    ``dst_ptrs`` the device addresses of item ``lo`` in every rank's buffer, own rank first."""

    is_cuda = True

    def __init__(self, owner, lo, hi):
        if not (0 <= lo < hi <= owner.shape[0]):
            raise ValueError("bad slice [%d, %d) of %d items" % (lo, hi, owner.shape[0]))
        self.owner, self.lo, self.hi = owner, lo, hi
        self.tensor = owner.tensor[lo:hi]
        self.dst_ptrs = owner.slice_ptrs(lo)
        self.shape = self.tensor.shape
        self.dtype = self.tensor.dtype
        self.device = self.tensor.device

    def push(self):
        """Copies the local view into the same items of every peer's buffer (device-to-device
        copies on the current stream; stores into peer memory only).  For kernels that have a
        single destination."""
        for r in self.owner.peer_order()[1:]:
            self.owner.view_of(r)[self.lo:self.hi].copy_(self.tensor, non_blocking=True)


class PeerGatheredOutput(object):
    """A ``[batch, *item_shape]`` output buffer present on every rank and writable by every rank.

    ``slice(lo, hi)`` is what a rank passes as the output of its module call; ``slice_ptrs(lo)``
    gives, own rank first, the device address of batch item ``lo`` in each rank's buffer - the
    destination list of ``backend.bgemm_bf16_multi``.  ``barrier()`` must follow the launch on
    the same stream before any rank reads the gathered result: it orders every rank's stores
    before every rank's reads.  ``close()`` drops the buffer; call it (on every rank, after a
    barrier) before the process group goes away.
    """

    def __init__(self, batch, *item_shape, dtype=torch.bfloat16, group=None):
        disable_symm_mem_multicast()  # before the rendezvous: plain peer pointers are all that is used
        if item_shape and isinstance(item_shape[-1], torch.dtype):  # (batch, m, n, dtype) spelling
            dtype, item_shape = item_shape[-1], item_shape[:-1]
        if not dist.is_initialized():
            raise RuntimeError("torch.distributed is not initialised")
        import torch.distributed._symmetric_memory as symm_mem
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.shape = (int(batch),) + tuple(int(x) for x in item_shape)
        self.device = torch.device("cuda", torch.cuda.current_device())
        self.tensor = symm_mem.empty(*self.shape, dtype=dtype, device=self.device)
        self.handle = symm_mem.rendezvous(self.tensor, self.group)
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        items = 1
        for x in self.shape[1:]:
            items *= x
        self.item_bytes = items * self.tensor.element_size()
        self._views = {}
        if len(self.ptrs) != self.world:
            raise RuntimeError("symmetric memory gave %d buffers for %d ranks" % (len(self.ptrs), self.world))

    def peer_order(self):
        # own buffer first, then the peers starting with the next rank: at any moment the ranks'
        # stores are spread over different receivers instead of all aiming at rank 0 first
        return [(self.rank + k) % self.world for k in range(self.world)]

    def slice_ptrs(self, lo):
        return [self.ptrs[r] + lo * self.item_bytes for r in self.peer_order()]

    def slice(self, lo, hi):
        return PeerSlice(self, lo, hi)

    def view_of(self, rank):
        """Rank ``rank``'s buffer as a tensor of this device (a mapping of the peer's memory)."""
        if rank == self.rank:
            return self.tensor
        if rank not in self._views:
            self._views[rank] = self.handle.get_buffer(rank, self.shape, self.tensor.dtype)
        return self._views[rank]

    def barrier(self):
        self.handle.barrier()

    def close(self):
        self._views.clear()
        self.handle = None
        self.tensor = None


GATHER_MODES = ("fused", "push", "nccl")


class ShardedOp(object):
    """One registered operator run batch-sharded through the task interface.

    builder : a task builder whose first argument is the batch (``task.batch_gemm``,
              ``task.conv2d``, ``task.depthwise_conv2d``)
    args    : the builder's arguments for the *whole* batch (``args[0]`` = batch)
    gather  : "fused" | "push" | "nccl" (see the module docstring); under "fused" an operator whose
              kernel writes one destination (conv2d) is pushed after the launch instead
    Every rank plans and builds the Task of its slice (``Task -> schedule_with_config ->
    build``) and calls ``func(*local_inputs, output)``; ``output`` is a ``PeerSlice`` (fused,
    push) or a local tensor followed by one all-gather (nccl).  ``__call__`` returns the gathered
    tensor, complete on every rank once the returned work has been synchronised.
    """

    def __init__(self, category, name, builder, args, gather="fused", knobs=None, precision=None, group=None):
        from .runtime import build, torch_dtype
        from .scheduler import schedule_with_config
        from .task import Task, register_task
        from .templates import knobs_to_config
        from .utils import Config
        if gather not in GATHER_MODES:
            raise ValueError("gather must be one of %s" % (GATHER_MODES,))
        self.group = group
        # without a process group the operator runs on this GPU alone (world size 1)
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.batch = int(args[0])
        if self.batch % self.world:
            raise ValueError("batch %d is not a multiple of the world size %d" % (self.batch, self.world))
        self.lo, self.hi = shard_range(self.batch, self.world, self.rank)
        self.local = self.hi - self.lo
        dev_id = torch.cuda.current_device() if torch.cuda.is_available() else 0
        task = Task(category, name, builder, (self.local,) + tuple(args[1:]), "cuda", dev_id)
        register_task(task)
        self.task = task
        ops, bufs = task.func(*task.args)
        op_lst_len = 1 if ops[0].kind in ("gemm", "batch_gemm", "gemm_int8") else 2  # conv graphs: pad + conv
        op_cfg = knobs_to_config(knobs, ops[0]) if knobs else {}
        configs = Config([{}] * (op_lst_len - 1) + [op_cfg], None)
        s, self.bufs = schedule_with_config(task.key, configs, precision=precision)
        self.func = build(s, self.bufs, "cuda")
        self.kind = ops[0].kind
        out_buf = self.bufs[-1]
        self.out_shape = (self.batch,) + tuple(int(x) for x in out_buf.shape[1:])
        self.out_dtype = torch_dtype(out_buf.dtype)
        self.gather = gather if self.world > 1 else "local"
        self.peer_out = None
        self.out_full = None
        self.out_local = None
        self._sharder = None
        self._needs_push = False
        device = torch.device("cuda", dev_id) if torch.cuda.is_available() else torch.device("cpu")
        if self.gather in ("fused", "push"):
            self.peer_out = PeerGatheredOutput(*self.out_shape, dtype=self.out_dtype, group=group)
            self.out_full = self.peer_out.tensor
            self._slice = self.peer_out.slice(self.lo, self.hi)
        elif self.gather == "nccl":
            self._sharder = BatchSharded(self.batch, group)
            self.out_full = torch.empty(self.out_shape, dtype=self.out_dtype, device=device)
            self.out_local = torch.empty((self.local,) + self.out_shape[1:], dtype=self.out_dtype, device=device)
        else:
            self.out_full = torch.empty(self.out_shape, dtype=self.out_dtype, device=device)

    def launch(self, *local_inputs):
        """The kernels only (compute, plus the stores into the peers for the fused form)."""
        if self.gather == "fused":
            self.func(*local_inputs, self._slice)
            self._needs_push = not self.func.pushed_by_kernel
        elif self.gather == "push":
            self.func(*local_inputs, self._slice.tensor)
            self._needs_push = True
        elif self.gather == "nccl":
            self.func(*local_inputs, self.out_local)
        else:
            self.func(*local_inputs, self.out_full)

    def finish(self):
        """What returns the output to every rank after ``launch``."""
        if self.gather in ("fused", "push") and self._needs_push:
            self._slice.push()
        if self.gather in ("fused", "push"):
            self.peer_out.barrier()
        elif self.gather == "nccl":
            self._sharder.gather(self.out_local, self.out_full)

    def __call__(self, *local_inputs):
        self.launch(*local_inputs)
        self.finish()
        return self.out_full

    def check(self):
        self.func.check()

    def close(self):
        if self.peer_out is not None:
            self.peer_out.close()
            self.peer_out = None
        self.out_full = None
