"""The reference-facing path on a GPU: Task -> schedule_with_config / schedule -> build ->
callable, the timing interface, and the measurer (host-side failure handling included)."""
import json

import numpy as np
import pytest
import torch

from oracle import ft_oracle as O

pytestmark = pytest.mark.gpu


def dev(x):
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


def test_readme_flow_gemm(native_lib):
    """README.md:131-158 with this backend: key -> schedule_with_config -> build -> func(*arrays)."""
    from flextensor_b200.runtime import build
    from flextensor_b200.scheduler import schedule_with_config
    from flextensor_b200.task import Task
    from flextensor_b200.utils import Config
    key = Task("gemm", "gemm", None, (1024, 1024, 1024), "cuda", 0).key
    s, bufs = schedule_with_config(key, Config([{}], None))
    func = build(s, bufs, "cuda")
    a, b = O.gemm_inputs(1024, 1024, 1024, seed=0)
    c = torch.zeros(1024, 1024, device="cuda")
    func(dev(a), dev(b), c)
    func.check()
    assert O.normalised_error(c.cpu().numpy(), O.gemm(a, b)) <= O.TOLERANCE["gemm_f32_3xtf32"]
    res = func.time_evaluator(func.entry_name, None, number=5)(dev(a), dev(b), c)
    assert 0 < res.mean < 1e-2
    assert json.loads(func.imported_modules[0].get_source())["steps"][0]["op"] == "gemm"
    with pytest.raises(ValueError):
        func(dev(a), dev(b))
    with pytest.raises(TypeError):
        func(dev(a), dev(b), c.double())


def test_captured_call_replays(native_lib):
    """A call frozen into a CUDA graph follows the contents of its buffers."""
    from flextensor_b200.runtime import build
    from flextensor_b200.scheduler import schedule_with_config
    from flextensor_b200.utils import Config
    key = "conv2d_depthwise_(1, 256, 56, 56, 1, 3, 1, 1, 1)_cuda(0)"
    s, bufs = schedule_with_config(key, Config([{}, {}], None))
    func = build(s, bufs)
    x, w = O.depthwise_inputs(1, 256, 56, 56, 1, 3, 3, seed=2)
    xd, wd, out = dev(x), dev(w), torch.zeros(1, 256, 56, 56, device="cuda")
    call = func.capture(xd, wd, out)
    x2, _ = O.depthwise_inputs(1, 256, 56, 56, 1, 3, 3, seed=99)
    xd.copy_(dev(x2))
    out.zero_()
    call.replay()
    torch.cuda.synchronize()
    assert O.normalised_error(out.cpu().numpy(), O.depthwise_conv2d_nchw(x2, w, None, 1, 1, 1)) <= 1e-5


def test_module_conv_depthwise_int8_bf16(native_lib):
    from flextensor_b200.runtime import build
    from flextensor_b200.scheduler import schedule_with_config, schedule_with_config_ops
    from flextensor_b200.ir import placeholder
    from flextensor_b200.nn import ops
    from flextensor_b200.utils import Config
    key = "conv2d_res_b13_(1, 64, 56, 56, 64, 3, 1, 1, 1, 1)_cuda(0)"
    s, bufs = schedule_with_config(key, Config([{}, {}], {"inline": [[1, 0]]}))
    x, w = O.conv2d_inputs(1, 64, 56, 56, 64, 3, 3, seed=1)
    out = torch.zeros(1, 64, 56, 56, device="cuda")
    func = build(s, bufs)
    func(dev(x), dev(w), out)
    func.check()
    assert O.normalised_error(out.cpu().numpy(), O.conv2d_nchw(x, w, None, 1, 1, 1)) <= O.TOLERANCE["conv2d_tf32"]
    # conv with bias: three stages in the graph, one kernel
    xi, wi, bi = placeholder((2, 8, 10, 10)), placeholder((12, 8, 3, 3)), placeholder((12,))
    yo = ops.conv2d_nchw(xi, wi, bi, stride=1, padding=1)
    plan, bufs = schedule_with_config_ops([yo.op], [xi, wi, bi, yo], Config([], None), precision="3xtf32")
    x, w = O.conv2d_inputs(2, 8, 10, 10, 12, 3, 3, seed=7)
    b = np.linspace(-1, 1, 12).astype(np.float32)
    out = torch.zeros(2, 12, 10, 10, device="cuda")
    plan.build()(dev(x), dev(w), dev(b), out)
    assert O.normalised_error(out.cpu().numpy(), O.conv2d_nchw(x, w, b, 1, 1, 1)) <= O.TOLERANCE["conv2d_3xtf32"]
    # depthwise
    key = "conv2d_depthwise_(1, 256, 56, 56, 1, 3, 1, 1, 1)_cuda(0)"
    s, bufs = schedule_with_config(key, Config([{}, {}], None))
    x, w = O.depthwise_inputs(1, 256, 56, 56, 1, 3, 3, seed=2)
    out = torch.zeros(1, 256, 56, 56, device="cuda")
    build(s, bufs)(dev(x), dev(w), out)
    assert O.normalised_error(out.cpu().numpy(), O.depthwise_conv2d_nchw(x, w, None, 1, 1, 1)) <= 1e-5
    # int8
    key = "gemm_gemm_int8_(256, 512, 384)_cuda(0)"
    s, bufs = schedule_with_config(key, Config([{}], None))
    a, b = O.gemm_int8_inputs(256, 384, 512, seed=4)
    c = torch.zeros(256, 384, device="cuda", dtype=torch.int32)
    build(s, bufs)(dev(a), dev(b), c)
    assert (c.cpu().numpy() == O.gemm_int8(a, b)).all()
    # bf16 batched
    key = "gemm_batch_gemm_(4, 256, 512, 384)_cuda(0)"
    s, bufs = schedule_with_config(key, Config([{}], None))
    items = [O.batch_gemm_item(i, 256, 384, 512) for i in range(4)]
    a = np.stack([i[0] for i in items])
    b = np.stack([i[1] for i in items])
    c = torch.zeros(4, 256, 384, device="cuda", dtype=torch.bfloat16)
    build(s, bufs)(dev(a).bfloat16(), dev(b).bfloat16(), c)
    assert O.bf16_output_ok(c.float().cpu().numpy(), O.batch_gemm(a, b))


def test_search_on_device_in_process(native_lib):
    """A short real search: candidates are measured on the GPU (no compile per candidate)."""
    from flextensor_b200 import scheduler as S
    from flextensor_b200.measure import InProcessMeasurer
    from flextensor_b200.runtime import build
    S.VERBOSE = False
    np.random.seed(0)
    torch.manual_seed(0)
    measurer = InProcessMeasurer(0)
    key = "gemm_batch_gemm_(8, 1024, 1024, 1024)_cuda(0)"
    plan, bufs, configs = S.schedule(key, op_trial=3, op_stop=2, timeout=10, parallel=1, number=3, measurer=measurer)
    assert plan.steps[0].knobs["tile_n"] in (64, 128, 256, 512)
    items = [O.batch_gemm_item(i, 1024, 1024, 1024) for i in range(2)]
    a = torch.stack([dev(i[0]).bfloat16() for i in items] * 4)
    b = torch.stack([dev(i[1]).bfloat16() for i in items] * 4)
    c = torch.zeros(8, 1024, 1024, device="cuda", dtype=torch.bfloat16)
    build(plan, bufs)(a, b, c)
    assert O.bf16_output_ok(c[1].float().cpu().numpy(), O.gemm(items[1][0], items[1][1], out_dtype=np.float64))


def test_gpu_pool_measurer_and_failures(native_lib):
    """One worker per GPU; a candidate the library rejects scores inf, the pool keeps working."""
    from flextensor_b200.measure import GpuPoolMeasurer
    from flextensor_b200.templates import knobs_to_config
    from flextensor_b200.task import TASK_TABLE
    from flextensor_b200.utils import Config
    key = "gemm_batch_gemm_(4, 256, 512, 384)_cuda(0)"
    op = TASK_TABLE[key].func(*TASK_TABLE[key].args)[0][0]
    good = Config([knobs_to_config({"tile_n": 128, "cluster": 1, "stages": 3}, op)], None)
    bad = Config([knobs_to_config({"tile_n": 256, "cluster": 1, "stages": 8}, op)], None)  # over the smem budget
    pool = GpuPoolMeasurer(devices=[0])
    try:
        res = pool([(key, good, None), (key, bad, None), (key, good, None)], number=3, timeout=60, parallel=1)
    finally:
        pool.close()
    assert 0 < res[0] < 100 and res[1] == float("inf") and 0 < res[2] < 100


def test_conv_filter_is_packed_once_per_weight_tensor(native_lib):
    """The second call with the same weight tensor finds the packed filter in the workspace (the
    layout pass then only copies the input) and gives the same bits; a modified or another weight
    tensor is packed again; every algorithm's filter layout goes through the same path."""
    from flextensor_b200 import backend as B
    from flextensor_b200.runtime import build
    from flextensor_b200.scheduler import schedule_with_config
    from flextensor_b200.task import Task, conv2d, register_task
    from flextensor_b200.templates import knobs_to_config
    from flextensor_b200.utils import Config
    for args, knobs in (((2, 32, 28, 28, 48, 3, 1, 1, 1, 1), {"algo": 2}),        # slab kernel
                        ((2, 40, 20, 24, 48, 3, 2, 1, 1, 1), {"algo": 1}),        # per-tap lowering
                        ((1, 3, 64, 64, 16, 7, 2, 3, 1, 1), {"algo": 4}),         # im2col rows
                        ((2, 64, 14, 14, 32, 1, 1, 0, 1, 1), {"algo": 3}),        # GEMM on the NCHW tensors: no packing
                        ((2, 18, 15, 16, 12, 3, 1, 1, 1, 6), {"algo": 1})):       # groups of 3 channels
        task = Task("conv2d", "packonce", conv2d, args, "cuda", 0)
        register_task(task)
        op = task.func(*task.args)[0][0]
        s, bufs = schedule_with_config(task.key, Config([{}, knobs_to_config(knobs, op)], None))
        func = build(s, bufs)
        n, c, h, w, k, r, stride, pad, dil, groups = args
        x, wt = O.conv2d_inputs(n, c, h, w, k, r, r, groups=groups, seed=81)
        want = O.conv2d_nchw(x, wt, None, stride, pad, dil, groups)
        xd, wd = dev(x), dev(wt)
        out1 = torch.full(want.shape, float("nan"), device="cuda")
        out2 = torch.full(want.shape, float("nan"), device="cuda")
        func(xd, wd, out1)
        assert func._packed, "first call records the packed weight"
        func(xd, wd, out2)                       # packed filter reused
        func.check()
        assert torch.equal(out1, out2)
        assert O.normalised_error(out2.cpu().numpy(), want) <= O.TOLERANCE["conv2d_tf32"], args
        wd.mul_(2.0)                             # in-place change bumps the version: packed again
        func(xd, wd, out2)
        func.check()
        assert O.normalised_error(out2.cpu().numpy(), 2.0 * want) <= O.TOLERANCE["conv2d_tf32"], args
        wd2 = dev(-wt)                           # another tensor: packed again
        func(xd, wd2, out2)
        func(xd, wd2, out1)
        func.check()
        assert torch.equal(out1, out2)
        assert O.normalised_error(out1.cpu().numpy(), -want) <= O.TOLERANCE["conv2d_tf32"], args


@pytest.mark.parametrize("args", [(2, 24, 200, 36, 9, 1, 4, 1, 3), (1, 16, 333, 8, 3, 2, 1, 2, 1),
                                  (3, 64, 196, 128, 1, 1, 0, 1, 1)])
def test_conv1d_task_runs_on_the_conv2d_kernels(native_lib, args):
    """conv1d (flextensor/nn/ops.py:293-351) through Task -> schedule_with_config -> build."""
    from flextensor_b200.runtime import build
    from flextensor_b200.scheduler import schedule_with_config
    from flextensor_b200.task import Task, conv1d, register_task
    from flextensor_b200.utils import Config
    n, c, length, k, k_len, stride, pad, dil, groups = args
    task = Task("conv1d", "conv1d", conv1d, args, "cuda", 0)
    register_task(task)
    s, bufs = schedule_with_config(task.key, Config([{}, {}], None))
    func = build(s, bufs)
    rng = np.random.default_rng(83)
    x = rng.standard_normal((n, c, length)).astype(np.float32)
    w = rng.standard_normal((k, c // groups, k_len)).astype(np.float32)
    want = O.conv1d(x, w, None, stride, pad, dil, groups)
    out = torch.full(want.shape, float("nan"), device="cuda")
    assert tuple(bufs[-1].shape) == want.shape
    func(dev(x), dev(w), out)
    func.check()
    assert O.normalised_error(out.cpu().numpy(), want) <= O.TOLERANCE["conv2d_tf32"]


def test_packed_1x1_and_gemm_conv2d_tasks(native_lib):
    from flextensor_b200.runtime import build
    from flextensor_b200.scheduler import schedule_with_config
    from flextensor_b200.task import Task, conv2d_1x1_packed, gemm_conv2d, register_task
    from flextensor_b200.utils import Config
    # out[b,k,i] = sum_rc A[b,rc,i] * B[k,rc]  (flextensor/task.py:168-173)
    task = Task("conv2d", "1x1-packed", conv2d_1x1_packed, (5, 48, 14, 14, 72, 1), "cuda", 0)
    register_task(task)
    s, bufs = schedule_with_config(task.key, Config([{}], None))
    func = build(s, bufs)
    rng = np.random.default_rng(84)
    a = rng.standard_normal((5, 48, 196)).astype(np.float32)
    b = rng.standard_normal((72, 48)).astype(np.float32)
    want = O.conv2d_1x1_packed(a, b)
    out = torch.full(want.shape, float("nan"), device="cuda")
    func(dev(a), dev(b), out)
    func.check()
    assert O.normalised_error(out.cpu().numpy(), want) <= O.TOLERANCE["conv2d_tf32"]
    # the im2col -> GEMM -> col2img definition gives the conv2d numbers (flextensor/nn/ops.py:982-1044)
    args = (2, 12, 13, 16, 18, 3, 2, 1, 1, 3)
    task = Task("gemm_conv2d", "t", gemm_conv2d, args, "cuda", 0)
    register_task(task)
    s, bufs = schedule_with_config(task.key, Config([{}, {}], None))
    func = build(s, bufs)
    x, w = O.conv2d_inputs(2, 12, 13, 16, 18, 3, 3, groups=3, seed=85)
    want = O.conv2d_nchw(x, w, None, 2, 1, 1, 3)
    out = torch.full(want.shape, float("nan"), device="cuda")
    func(dev(x), dev(w), out)
    func.check()
    assert O.normalised_error(out.cpu().numpy(), want) <= O.TOLERANCE["conv2d_tf32"]


@pytest.mark.parametrize("case", [dict(n=2, c=32, h=20, w=24, k=48, r=3, stride=1, pad=1, groups=1),      # slab kernel
                                  dict(n=2, c=24, h=15, w=16, k=36, r=3, stride=2, pad=1, groups=3),      # per-tap, groups
                                  dict(n=1, c=16, h=9, w=7, k=8, r=3, stride=1, pad=0, groups=1)])        # per-thread stores
def test_conv_bias_relu_chain_is_one_kernel(native_lib, case):
    """pad -> conv2d -> bias -> ReLU planned from the op graph: one layout pass and one conv kernel whose
    epilogue adds the bias and clamps at zero (flextensor/nn/ops.py:474-478 is the bias stage)."""
    from flextensor_b200 import backend as B
    from flextensor_b200.ir import placeholder
    from flextensor_b200.nn import conv2d_nchw, relu
    from flextensor_b200.runtime import build
    from flextensor_b200.scheduler import schedule_with_config_ops
    from flextensor_b200.utils import Config
    n, c, h, w, k, r = case["n"], case["c"], case["h"], case["w"], case["k"], case["r"]
    img = placeholder((n, c, h, w))
    wt = placeholder((k, c // case["groups"], r, r))
    bias = placeholder((k,))
    out = relu(conv2d_nchw(img, wt, bias, stride=case["stride"], padding=case["pad"], groups=case["groups"]))
    s, bufs = schedule_with_config_ops([out.op], [img, wt, bias, out], Config([{}, {}, {}, {}], None))
    assert [st.op.kind for st in s.steps] == ["conv2d"] and s.steps[0].knobs["relu"] == 1
    func = build(s, bufs)
    x, wv = O.conv2d_inputs(n, c, h, w, k, r, r, groups=case["groups"], seed=86)
    bv = np.random.default_rng(87).standard_normal(k).astype(np.float32)
    want = np.maximum(O.conv2d_nchw(x, wv, bv, case["stride"], case["pad"], 1, case["groups"]), 0.0)
    got = torch.full(want.shape, float("nan"), device="cuda")
    before = B.launch_count()
    func(dev(x), dev(wv), dev(bv), got)
    func.check()
    assert B.launch_count() - before == 2
    got = got.cpu().numpy()
    assert (got >= 0).all() and (got == 0).any()
    assert O.normalised_error(got, want) <= O.TOLERANCE["conv2d_tf32"]


def test_depthwise_bias_relu_chain(native_lib):
    from flextensor_b200.ir import placeholder
    from flextensor_b200.nn import depthwise_conv2d_nchw, relu
    from flextensor_b200.runtime import build
    from flextensor_b200.scheduler import schedule_with_config_ops
    from flextensor_b200.utils import Config
    img, wt, bias = placeholder((2, 16, 28, 28)), placeholder((16, 2, 3, 3)), placeholder((32,))
    out = relu(depthwise_conv2d_nchw(img, wt, bias, stride=1, padding=1))
    s, bufs = schedule_with_config_ops([out.op], [img, wt, bias, out], Config([{}, {}, {}, {}], None))
    func = build(s, bufs)
    x, wv = O.depthwise_inputs(2, 16, 28, 28, 2, 3, 3, seed=88)
    bv = np.random.default_rng(89).standard_normal(32).astype(np.float32)
    want = np.maximum(O.depthwise_conv2d_nchw(x, wv, bv, 1, 1, 1), 0.0)
    got = torch.full(want.shape, float("nan"), device="cuda")
    func(dev(x), dev(wv), dev(bv), got)
    func.check()
    assert O.normalised_error(got.cpu().numpy(), want) <= O.TOLERANCE["depthwise_f32"]
