"""Shared pieces of the drivers: timing of a planned task, the parity check behind
``--check`` and the argument parser.

Mirrors flextensor/optimize/common.py: ``evaluate`` (:17-60) builds and times a plan,
``test`` (:63-82) replays a logged config and, with ``check_result``, compares the kernel
result with a default-schedule CPU result at rtol 1e-3; ``init_arg_parser`` (:85-114) keeps
the reference's flags (the RPC ones are accepted and ignored: there are no remote boards).
The CPU result of the check is computed here with torch on the host - the role the
default-schedule llvm build plays in the reference.
"""
import numpy as np

from ..measure import make_inputs
from ..runtime import build
from ..scheduler import schedule_with_config, flatten_graph
from ..task import TASK_TABLE
from ..utils import test_allclose, to_tuple

LIB_DIR = "."


def host_result(ops, bufs, arrays):
    """Output of the task's op graph computed on the host CPU with torch (float64 accumulate for
    floating point, exact integers for int8)."""
    import torch
    import torch.nn.functional as F
    op_lst, _ = flatten_graph(ops)
    values = {id(buf): arr.detach().cpu() for buf, arr in zip(bufs, arrays)}

    def val(t):
        return values[id(t)]

    for op in op_lst:
        ins = op.input_tensors
        if op.kind == "pad2d":
            p = op.attrs["padding"]  # (first axis before, after, ..., last axis before, after)
            last_first = [v for i in range(len(p) - 2, -2, -2) for v in (p[i], p[i + 1])]
            if op.attrs.get("layout") == "nhwc":
                last_first = [0, 0] + last_first   # (h, w) padding of [N, H, W, C]
            values[id(op.output(0))] = F.pad(val(ins[0]).double(), last_first)
        elif op.kind == "conv2d":
            x, w = val(ins[0]).double(), val(ins[1]).double()
            form = op.attrs.get("form")
            if form == "conv1d":
                res = F.conv1d(x, w, None, op.attrs["stride"][1], 0, op.attrs["dilation"][1], op.attrs["groups"])
            elif form == "packed_1x1":
                res = torch.einsum("bci,kc->bki", x, w)
            elif form == "nhwc":
                res = F.conv2d(x.permute(0, 3, 1, 2), w, None, op.attrs["stride"], 0, op.attrs["dilation"],
                               op.attrs["groups"]).permute(0, 2, 3, 1).contiguous()
            elif form == "conv3d":
                res = F.conv3d(x, w, None, op.attrs["stride"], 0, op.attrs["dilation"], op.attrs["groups"])
            else:
                res = F.conv2d(x, w, None, op.attrs["stride"], 0, op.attrs["dilation"], op.attrs["groups"])
            values[id(op.output(0))] = res
        elif op.kind == "depthwise_conv2d":
            x, w = val(ins[0]).double(), val(ins[1]).double()
            c, f, r, s = w.shape
            values[id(op.output(0))] = F.conv2d(x, w.reshape(c * f, 1, r, s), None, op.attrs["stride"], 0,
                                                op.attrs["dilation"], c)
        elif op.kind == "bias_add":
            x = val(ins[0])
            axis = op.attrs.get("axis", 1)
            values[id(op.output(0))] = x + val(ins[1]).double().reshape([1] * axis + [-1] + [1] * (x.dim() - axis - 1))
        elif op.kind == "relu":
            values[id(op.output(0))] = val(ins[0]).clamp(min=0)
        elif op.kind in ("gemm", "batch_gemm", "gemm_int8"):
            a, b = val(ins[0]).double(), val(ins[1]).double()
            if op.attrs["transposeA"]:
                a = a.transpose(-1, -2)
            if op.attrs["transposeB"]:
                b = b.transpose(-1, -2)
            values[id(op.output(0))] = a @ b
        else:
            raise RuntimeError("no host rule for op kind %r" % (op.kind,))
    return values[id(bufs[-1])].double().numpy()


def evaluate(name, s, bufs, target, dev_id, number=10, rpc_info=None, result_generator=None):
    """Build the plan, run it once (optionally checking the result), then time it; milliseconds."""
    import torch
    time_cost = float("inf")
    try:
        device = torch.device("cuda", dev_id)
        with torch.cuda.device(device):
            arrays = make_inputs(bufs, device, low=-10.0, high=10.0)
            func = build(s, bufs, target)
            func(*arrays)
            func.check()
            if result_generator is not None:
                print("Test correctness...")
                expected = result_generator(arrays)
                result = arrays[-1].double().cpu().numpy()
                scale = max(float(np.abs(expected).max()), 1e-30)
                test_allclose(result / scale, expected / scale, rtol=1e-3, print_diff=True)
            evaluator = func.time_evaluator(func.entry_name, None, number=number)
            time_cost = evaluator(*arrays).mean * 1e3
    except Exception as exc:  # as in the reference: report and return inf
        print(exc)
    return time_cost


def test(task_key, configs, dev_id=None, rpc_info=None, check_result=False):
    task = TASK_TABLE[task_key]
    result_generator = None
    if check_result:
        def _generator(arrays):
            ops, bufs = task.func(*task.args)
            return host_result(ops, bufs, arrays)
        result_generator = _generator
    s, bufs = schedule_with_config(task_key, configs)
    dev_id = dev_id if dev_id is not None else task.dev_id
    time_cost = evaluate(task_key, s, bufs, task.target, dev_id, 100, rpc_info, result_generator)
    print(task_key, "use", time_cost, "ms")
    print()
    return time_cost


test.__test__ = False  # not a pytest test


def init_arg_parser(parser):
    parser.add_argument("-f", "--from_", help="From which shape", type=int, default=0)
    parser.add_argument("-t", "--to", help="To which shape", type=int, default=-1)
    parser.add_argument("-l", "--log", help="Log file name", type=str, default="")
    parser.add_argument("--test", help="test file name", type=str, default="")
    parser.add_argument("--trials", help="number of trials for op", type=int, default=100)
    parser.add_argument("--target", help="target device type (only 'cuda' is built)", type=str, default="cuda")
    parser.add_argument("--device", help="target device number", type=int, default=0)
    parser.add_argument("--timeout", help="timeout", type=int, default=4)
    parser.add_argument("--parallel", help="GPUs used to measure candidates", type=int, default=1)
    parser.add_argument("--use_model", help="use performance model", action="store_true")
    parser.add_argument("--method", help="how to schedule", type=str, default="searching")
    parser.add_argument("--slevel", type=int, default=4)
    parser.add_argument("--rlevel", type=int, default=3)
    parser.add_argument("--force_inline", action="store_true")
    parser.add_argument("--check", action="store_true")
    parser.add_argument("--seed", type=int, default=None)
    parser.add_argument("--precision", type=str, default=None, choices=[None, "tf32", "3xtf32"])
    # accepted for command-line compatibility with the reference; unused (no remote boards)
    parser.add_argument("--host", type=str, default="0.0.0.0")
    parser.add_argument("--target_host", type=str, default="llvm")
    parser.add_argument("--device_key", type=str, default="")
    parser.add_argument("--use_rpc", type=str, choices=["server", "tracker"])
    parser.add_argument("--fcompile", type=str, choices=["ndk"])
    parser.add_argument("--port", type=int, default=9190)
