"""Batch-sharded execution over several GPUs of one node.

The reference runs every operator on one device (its only multi-device notion is the
``dev_id`` a task is pinned to, flextensor/task.py:226).  Batched GEMM and batched conv
shard naturally along the batch axis: items are independent, so each rank computes its
contiguous slice with the single-GPU kernels and no data-path exchange; the only
collective is one all-gather that returns the full output to every rank (NCCL over
NVLink via ``torch.distributed``).  ``run`` can overlap that gather with compute by
splitting the local slice into chunks: chunk i is gathered on a side stream while chunk
i+1 is computed.

``PeerGatheredOutput`` removes the collective altogether: the gathered output lives in
symmetric memory (every rank maps every rank's buffer over NVLink) and the GEMM epilogue writes
each finished slab of a rank's slice into all ranks' buffers with bulk tensor stores
(``ftb_bgemm_bf16_multi``), so the transfer overlaps the math tile by tile; what is left of the
all-gather is one barrier after the kernel.  Plain peer stores only (no multicast objects).

One process per GPU; ``torch.distributed`` must be initialised by the caller.
"""
import torch
import torch.distributed as dist


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


class PeerGatheredOutput(object):
    """A [batch, m, n] output buffer present on every rank and writable by every rank.

    ``slice_ptrs(lo)`` gives, own rank first, the device address of batch item ``lo`` in each
    rank's buffer - the destination list of ``backend.bgemm_bf16_multi``.  ``barrier()`` must
    follow the launch on the same stream before any rank reads the gathered result: it orders
    every rank's stores before every rank's reads.
    """

    def __init__(self, batch, m, n, dtype=torch.bfloat16, group=None):
        import torch.distributed._symmetric_memory as symm_mem
        if not dist.is_initialized():
            raise RuntimeError("torch.distributed is not initialised")
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.shape = (batch, m, n)
        self.tensor = symm_mem.empty(batch, m, n, dtype=dtype, device=torch.device("cuda", torch.cuda.current_device()))
        self.handle = symm_mem.rendezvous(self.tensor, self.group)
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.item_bytes = m * n * self.tensor.element_size()
        if len(self.ptrs) != self.world:
            raise RuntimeError("symmetric memory gave %d buffers for %d ranks" % (len(self.ptrs), self.world))

    def slice_ptrs(self, lo):
        # own buffer first, then the peers starting with the next rank: at any moment the ranks'
        # stores are spread over different receivers instead of all aiming at rank 0 first
        order = [(self.rank + k) % self.world for k in range(self.world)]
        return [self.ptrs[r] + lo * self.item_bytes for r in order]

    def barrier(self):
        self.handle.barrier()
