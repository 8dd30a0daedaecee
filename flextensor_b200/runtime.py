"""The runnable object that stands where ``tvm.build``'s output stood.

``KernelPlan`` is what ``schedule`` / ``schedule_with_config`` return as ``s``: the op graph,
the chosen configs and, per op, the kernel knobs derived from them.  ``build(s, bufs,
target)`` (or ``plan.build()``) gives a ``Module`` with the surface the reference's call
sites use on a ``tvm.runtime.Module``:

  func(*arrays)                              destination-passing, arrays in ``bufs`` order, output last
                                             (README.md:153-158, optimize/common.py:34-39)
  func.entry_name                            (measure.py:109)
  func.time_evaluator(name, ctx, number=n)   -> callable(*arrays) -> result with ``.mean`` in seconds
                                             (measure.py:109-110, optimize/common.py:47-48)
  func.imported_modules[0].get_source()      (test/naive_schedule_all.py:10-11)
  func.export_library(path)                  writes the plan as JSON; ``load_module(path)`` reads it back
                                             (measure.py:91,107) - the kernels themselves are pre-compiled

Arrays are CUDA ``torch.Tensor``s.  The output may instead be a ``sharded.PeerSlice`` - a rank's
slice of an output that every rank of a batch-sharded run holds: the kernel then writes its
result into every rank's copy (batched GEMM bf16 and depthwise conv2d do it themselves, store
by store; other operators write the local copy and leave the rest to ``PeerSlice.push``).  The padding stage of a conv graph never runs as a
kernel of its own: the conv kernels read out-of-image taps as zeros, so the graph-level
"inline" choice of the reference is always in effect; a bias stage is folded into the conv
epilogue.
"""
import json
import os

import torch

from . import backend
from .templates import config_to_knobs
from .utils import Config, to_tuple

_TORCH_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "int8": torch.int8, "int32": torch.int32}

DEFAULT_PRECISION = {"gemm": "3xtf32", "batch_gemm": "3xtf32", "conv2d": "tf32"}


def torch_dtype(name):
    return _TORCH_DTYPES[name]


class KernelStep(object):
    """One kernel launch of a plan: the op it serves, its knobs and where its operands come from."""

    def __init__(self, op, knobs, inputs, bias=None, out=None):
        self.op = op
        self.knobs = dict(knobs)
        self.inputs = inputs  # tensors of the graph (placeholders) feeding the kernel
        self.bias = bias
        self.out = out


class KernelPlan(object):
    def __init__(self, ops, op_lst, op_states, bufs, configs, target="cuda", op_pos=None, precision=None,
                 dev_id=0):
        self.ops = ops
        self.op_lst = op_lst
        self.op_states = op_states
        self.bufs = list(bufs)
        self.configs = configs
        self.target = target
        self.op_pos = op_pos
        self.precision = precision
        self.dev_id = dev_id
        self.steps = self._lower()

    def _config_of(self, index):
        lst = self.configs.op_config_lst
        return lst[index] if index < len(lst) and lst[index] else {}

    def _lower(self):
        """Fold pad / bias stages into their conv and translate configs to knobs."""
        steps = []
        index_of = {id(op): i for i, op in enumerate(self.op_lst)}
        consumed_bias = set()
        for i, op in enumerate(self.op_lst):
            if op.kind == "pad2d":
                continue  # read as zeros by the consuming conv kernel
            if op.kind in ("bias_add", "relu"):
                if id(op) in consumed_bias:
                    continue
                raise RuntimeError("a %s stage must follow a convolution" % op.kind)
            knobs = config_to_knobs(self._config_of(i), op)
            inputs = list(op.input_tensors)
            bias = None
            out = op.output(0)
            if op.kind in ("conv2d", "depthwise_conv2d"):
                padded = inputs[0]
                if getattr(padded.op, "kind", None) == "pad2d":
                    inputs[0] = padded.op.input_tensors[0]
                # a bias stage consuming this conv, and a ReLU consuming either, are folded into the epilogue
                for later in self.op_lst[i + 1:]:
                    if later.kind == "bias_add" and later.input_tensors[0] is out and bias is None:
                        bias = later.input_tensors[1]
                        out = later.output(0)
                        consumed_bias.add(id(later))
                    elif later.kind == "relu" and later.input_tensors[0] is out and not knobs.get("relu"):
                        knobs["relu"] = 1
                        out = later.output(0)
                        consumed_bias.add(id(later))
            if op.kind in DEFAULT_PRECISION and op.input_tensors[0].dtype == "float32":
                mode = self.precision or DEFAULT_PRECISION[op.kind]
                if mode not in ("tf32", "3xtf32"):
                    raise ValueError("precision must be 'tf32' or '3xtf32', got %r" % (mode,))
                knobs["fp32_mode"] = 1 if mode == "3xtf32" else 0
                if mode == "3xtf32":
                    knobs.pop("cluster", None)  # the split stage runs in single-CTA tiles only
            steps.append(KernelStep(op, knobs, inputs, bias=bias, out=out))
        return steps

    def build(self, target=None):
        return Module(self)

    def describe(self):
        return {"target": self.target, "configs": [self.configs.op_config_lst, self.configs.graph_config],
                "steps": [{"op": st.op.kind, "knobs": st.knobs} for st in self.steps]}


class _TimeResult(object):
    def __init__(self, results):
        self.results = list(results)
        self.mean = sum(self.results) / len(self.results)
        self.median = sorted(self.results)[len(self.results) // 2]
        self.min = min(self.results)
        self.max = max(self.results)


class Module(object):
    entry_name = "default_function"

    def __init__(self, plan):
        if plan.target != "cuda":
            raise RuntimeError("only target 'cuda' (sm_100a) can be built; got %r" % (plan.target,))
        backend.lib()  # fail loudly when the native library is missing
        self.plan = plan
        self.imported_modules = [self]
        self._status = None
        self._workspaces = {}
        self._peer_dst = {}
        self._conv_single_dst = {}
        self._packed = {}      # step -> (weight tensor, its version, workspace) whose packing the workspace holds
        self.pack_once = True  # conv2d: pack the filter on the first call only (see __call__)
        self.pushed_by_kernel = True  # False after a call whose PeerSlice output was written locally only

    # ------------------------------------------------------------ execution
    def _bind(self, arrays):
        bufs = self.plan.bufs
        if len(arrays) != len(bufs):
            raise ValueError("expected %d arrays (bufs order, output last), got %d" % (len(bufs), len(arrays)))
        table = {}
        self._peer_dst = {}
        for buf, arr in zip(bufs, arrays):
            if hasattr(arr, "dst_ptrs") and hasattr(arr, "tensor"):
                # a slice of a peer-gathered output: the local view stands for it in every check
                # below, and kernels that can write several destinations get the whole list
                self._peer_dst[id(buf)] = [int(p) for p in arr.dst_ptrs]
                arr = arr.tensor
            if not isinstance(arr, torch.Tensor) or not arr.is_cuda:
                raise TypeError("arrays must be CUDA torch tensors")
            if tuple(arr.shape) != to_tuple(buf.shape):
                raise ValueError("array of shape %s given for buffer %s" % (tuple(arr.shape), buf))
            if arr.dtype != torch_dtype(buf.dtype):
                raise TypeError("array of dtype %s given for buffer %s" % (arr.dtype, buf))
            table[id(buf)] = arr
        return table

    def _status_word(self, device):
        if self._status is None or self._status.device != device:
            self._status = backend.new_status(device)
        return self._status

    def _workspace(self, key, nbytes, device):
        ws = self._workspaces.get(key)
        if ws is None or ws.numel() < nbytes or ws.device != device:
            ws = torch.empty(max(nbytes, 1), dtype=torch.uint8, device=device)
            self._workspaces[key] = ws
        return ws

    def _filter_is_packed(self, idx, weight, ws):
        """Weights are constant per task: the filter is packed by the first call and found in the
        workspace by the next ones, for as long as the same weight tensor comes back unmodified
        (identity and torch's version counter; `invalidate()` after changing it behind torch's back,
        e.g. through a raw pointer).  Returns whether step ``idx`` may skip the packing."""
        seen = self._packed.get(idx)
        packed = (self.pack_once and seen is not None and seen[0] is weight and seen[1] == weight._version and
                  seen[2] is ws)
        if self.pack_once and not packed:
            self._packed[idx] = (weight, weight._version, ws)
        return packed

    def __call__(self, *arrays):
        table = self._bind(arrays)
        device = arrays[-1].device
        self.pushed_by_kernel = True
        status = self._status_word(device)
        for idx, step in enumerate(self.plan.steps):
            op = step.op
            try:
                ins = [table[id(t)] for t in step.inputs]
                out = table[id(step.out)]
            except KeyError:
                raise RuntimeError("every tensor a kernel touches must be one of bufs (intermediates are fused)")
            bias = table[id(step.bias)] if step.bias is not None else None
            cfg = step.knobs or None
            peers = self._peer_dst.get(id(step.out))  # every rank's copy of this step's output, own first
            if op.kind == "gemm":
                backend.gemm_f32(ins[0], ins[1], out, op.attrs["transposeA"], op.attrs["transposeB"], cfg=cfg,
                                 status=status)
            elif op.kind == "batch_gemm":
                if ins[0].dtype == torch.bfloat16 and peers and len(peers) > 1:
                    backend.bgemm_bf16_multi(ins[0], ins[1], peers, out.shape[1], out.shape[2],
                                             op.attrs["transposeA"], op.attrs["transposeB"],
                                             out_f32=out.dtype == torch.float32, cfg=cfg, status=status)
                    peers = None
                elif ins[0].dtype == torch.bfloat16:
                    backend.bgemm_bf16(ins[0], ins[1], out, op.attrs["transposeA"], op.attrs["transposeB"],
                                       cfg=cfg, status=status)
                else:
                    backend.bgemm_f32(ins[0], ins[1], out, op.attrs["transposeA"], op.attrs["transposeB"],
                                      cfg=cfg, status=status)
            elif op.kind == "gemm_int8":
                backend.gemm_s8(ins[0], ins[1], out, op.attrs["transposeA"], op.attrs["transposeB"], cfg=cfg,
                                status=status)
            elif op.kind == "conv2d" and op.attrs.get("form") == "conv3d":
                n, c, d, h, w = ins[0].shape
                k, _, t, r, s = ins[1].shape
                groups = op.attrs["groups"]
                ws = self._workspace(idx, backend.conv3d_workspace_bytes(n, c, d, h, w, k, t, r, s, groups), device)
                prepacked = self._filter_is_packed(idx, ins[1], ws)
                backend.conv3d_ncdhw_f32(ins[0], ins[1], out, bias, op.attrs["stride"], op.attrs["padding"],
                                         op.attrs["dilation"], groups, cfg=cfg, workspace=ws, status=status,
                                         prepacked=prepacked)
            elif op.kind == "conv2d" and op.attrs.get("form") == "nhwc":
                n, h, w, c = ins[0].shape
                k, _, r, s = ins[1].shape
                groups = op.attrs["groups"]
                ws = self._workspace(idx, backend.conv2d_nhwc_workspace_bytes(c, k, r, s, groups), device)
                prepacked = self._filter_is_packed(idx, ins[1], ws)
                backend.conv2d_nhwc_f32(ins[0], ins[1], out, bias, op.attrs["stride"], op.attrs["padding"],
                                        op.attrs["dilation"], groups, cfg=cfg, workspace=ws, status=status,
                                        prepacked=prepacked)
            elif op.kind == "conv2d":
                form = op.attrs.get("form")
                if form == "conv1d":        # [N,C,L] is a one-row image, the filter a one-row filter
                    ins = [ins[0].unsqueeze(2), ins[1].unsqueeze(2)]
                    out = out.unsqueeze(2)
                elif form == "packed_1x1":  # [N,C,HW] is a one-column image under a 1x1 filter
                    ins = [ins[0].unsqueeze(3), ins[1].view(ins[1].shape[0], ins[1].shape[1], 1, 1)]
                    out = out.unsqueeze(3)
                n, c, h, w = ins[0].shape
                k, _, r, s = ins[1].shape
                groups = op.attrs["groups"]
                ws = self._workspace(idx, backend.conv2d_workspace_bytes(n, c, h, w, k, r, s, groups), device)
                prepacked = self._filter_is_packed(idx, ins[1], ws)
                fused = False
                if peers and len(peers) > 1 and not self._conv_single_dst.get(idx):
                    try:
                        backend.conv2d_nchw_f32_multi(ins[0], ins[1], peers, bias, op.attrs["stride"],
                                                      op.attrs["padding"], op.attrs["dilation"], groups, cfg=cfg,
                                                      workspace=ws, status=status, prepacked=prepacked)
                        fused, peers = True, None
                    except backend.FtbError as exc:
                        if exc.code != -2:
                            raise
                        self._conv_single_dst[idx] = True  # this shape's kernel writes one destination
                if not fused:
                    backend.conv2d_nchw_f32(ins[0], ins[1], out, bias, op.attrs["stride"], op.attrs["padding"],
                                            op.attrs["dilation"], groups, cfg=cfg, workspace=ws, status=status,
                                            prepacked=prepacked)
            elif op.kind == "depthwise_conv2d":
                if peers and len(peers) > 1:
                    backend.dwconv2d_nchw_f32_multi(ins[0], ins[1], peers, bias, op.attrs["stride"],
                                                    op.attrs["padding"], op.attrs["dilation"], cfg=cfg, status=status)
                    peers = None
                else:
                    backend.dwconv2d_nchw_f32(ins[0], ins[1], out, bias, op.attrs["stride"], op.attrs["padding"],
                                              op.attrs["dilation"], cfg=cfg, status=status)
            else:
                raise RuntimeError("no kernel for op kind %r" % (op.kind,))
            if peers and len(peers) > 1:
                # this operator's kernel writes one destination: the caller still has to push the
                # local copy to the peers (sharded.PeerSlice.push)
                self.pushed_by_kernel = False

    def invalidate(self):
        """Forget packed filters: the next conv2d call packs its weights again."""
        self._packed.clear()

    def capture(self, *arrays):
        """Record one call on these arrays into a CUDA graph; returns an object whose ``replay()``
        re-runs it with a single launch from the host.

        For microsecond-sized operators the Python and launch cost of ``func(*arrays)`` (tens of
        microseconds) exceeds the kernels' own time; a serving loop that calls the operator on the
        same buffers every step replays the graph instead.  The arrays must stay alive and keep
        their addresses; their contents may change between replays.
        """
        stream = torch.cuda.current_stream()
        self(*arrays)  # first call outside the capture: one-time set-up (attributes, workspaces)
        stream.synchronize()
        self.check()
        side = torch.cuda.Stream(device=arrays[-1].device)
        side.wait_stream(stream)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                self(*arrays)
        stream.wait_stream(side)
        return CapturedCall(self, graph, arrays)

    def check(self):
        """Synchronise and raise if a kernel of this module reported a failed in-kernel wait."""
        if self._status is not None:
            backend.check_status(self._status)

    # ------------------------------------------------------------ timing
    def time_evaluator(self, func_name=None, ctx=None, number=10, repeat=1, min_repeat_ms=0, use_graph=True,
                       flush_l2=False, warmup=3):
        """Returns ``f(*arrays) -> result`` with ``result.mean`` in seconds per call.

        Device time from CUDA events on the current stream.  With ``use_graph`` the
        ``number`` back-to-back calls are captured once into a CUDA graph and replayed, so
        that host launch cost does not hide the kernels' own time for microsecond-sized ops.
        ``flush_l2`` writes a 256 MB scratch before every timed call (then each call is timed
        on its own and ``use_graph`` is ignored).
        """
        module = self

        def evaluator(*arrays):
            stream = torch.cuda.current_stream()
            for _ in range(max(warmup, 1)):
                module(*arrays)
            stream.synchronize()
            module.check()
            results = []
            if flush_l2:
                scratch = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=arrays[-1].device)
                for _ in range(repeat):
                    total = 0.0
                    for _ in range(number):
                        scratch.zero_()
                        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                        e0.record(stream)
                        module(*arrays)
                        e1.record(stream)
                        e1.synchronize()
                        total += e0.elapsed_time(e1)
                    results.append(total / number * 1e-3)
                module.check()
                return _TimeResult(results)
            graph = None
            if use_graph:
                side = torch.cuda.Stream(device=arrays[-1].device)
                side.wait_stream(stream)
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.stream(side):
                    with torch.cuda.graph(graph, stream=side):
                        for _ in range(number):
                            module(*arrays)
                stream.wait_stream(side)
                graph.replay()
                stream.synchronize()
            for _ in range(repeat):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
                if graph is not None:
                    graph.replay()
                else:
                    for _ in range(number):
                        module(*arrays)
                e1.record(stream)
                e1.synchronize()
                results.append(e0.elapsed_time(e1) / number * 1e-3)
            module.check()
            return _TimeResult(results)

        return evaluator

    # ------------------------------------------------------------ introspection / persistence
    def get_source(self, fmt="json"):
        """The plan (ops, configs, kernel knobs) as JSON text; the kernels are the pre-compiled
        ones of ``libftb200.so`` (sources under ``flextensor_b200/csrc``)."""
        return json.dumps(self.plan.describe(), indent=1)

    def export_library(self, path, fcompile=None):
        with open(path, "w") as fout:
            fout.write(self.get_source())


class CapturedCall(object):
    """A call of a ``Module`` frozen into a CUDA graph (see ``Module.capture``)."""

    def __init__(self, module, graph, arrays):
        self.module = module
        self.graph = graph
        self.arrays = arrays  # keeps the buffers alive

    def replay(self):
        self.graph.replay()

    __call__ = replay


def build(s, bufs=None, target="cuda", target_host=None, name="default_function"):
    """Counterpart of ``tvm.build(s, bufs, target)`` for a ``KernelPlan``."""
    if not isinstance(s, KernelPlan):
        raise TypeError("build() takes the plan returned by schedule()/schedule_with_config()")
    if target not in (None, "cuda"):
        raise RuntimeError("only target 'cuda' (sm_100a) can be built; got %r" % (target,))
    return s.build()


def load_module(path):
    """Reads back what ``export_library`` wrote (plan description only; rebuild with
    ``schedule_with_config`` to run it)."""
    with open(path, "r") as fin:
        return json.load(fin)
