"""conv3d (NCDHW) on the sm_100a per-tap conv kernel, through the C ABI and through the task API, against
the numpy oracle (oracle/ft_oracle.py:conv3d_ncdhw, which restates flextensor/nn/ops.py:689-751).

Tolerances are those of conv2d: normalised error <= 5e-3 single-pass TF32, <= 1e-4 3xTF32.
"""
import os
import random

import numpy as np
import pytest
import torch

from conftest import GOLDEN_DIR
from oracle import ft_oracle as O

pytestmark = pytest.mark.gpu

TOL = O.TOLERANCE


@pytest.fixture(scope="module")
def B(native_lib):
    from flextensor_b200 import backend
    assert backend.lib().ftb_device_check() == 0, "the current device is not sm_100"
    return backend


@pytest.fixture()
def status(B):
    st = B.new_status()
    yield st
    B.check_status(st)


def _triple(v):
    return (v, v, v) if isinstance(v, int) else tuple(v)


def run_conv3d(B, x, w, bias=None, stride=1, padding=0, dilation=1, groups=1, cfg=None, status=None, calls=1):
    stride, padding, dilation = _triple(stride), _triple(padding), _triple(dilation)
    n, c, d, h, wd = x.shape
    k, _, t, r, s = w.shape
    od = O.out_size(d, t, stride[0], padding[0], dilation[0])
    p = O.out_size(h, r, stride[1], padding[1], dilation[1])
    q = O.out_size(wd, s, stride[2], padding[2], dilation[2])
    out = torch.full((n, k, od, p, q), float("nan"), device="cuda")
    ws = torch.empty(B.conv3d_workspace_bytes(n, c, d, h, wd, k, t, r, s, groups), dtype=torch.uint8, device="cuda")
    cu = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    xd, wd_, bd = cu(x), cu(w), cu(bias) if bias is not None else None
    for i in range(calls):   # calls after the first find the filter packed in the workspace
        if i:
            out.fill_(float("nan"))
        B.conv3d_ncdhw_f32(xd, wd_, out, bd, stride, padding, dilation, groups, cfg=cfg, workspace=ws, status=status,
                           prepacked=i > 0)
    torch.cuda.synchronize()
    return out.cpu().numpy()


def _inputs(n, c, d, h, w, k, t, r, s, groups, seed):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((n, c, d, h, w)).astype(np.float32)
    wt = rng.standard_normal((k, c // groups, t, r, s)).astype(np.float32)
    return x, wt


def test_conv3d_golden(B, status):
    # the reference's own conv3d test case (flextensor/test/test_ops.py:187-214): 6 channels in 3 groups, 9 filters
    # of 3x3x3, stride 2, padding 1, dilation 2, bias
    g = np.load(os.path.join(GOLDEN_DIR, "conv3d_grouped.npz"))
    stride, pad, dil, groups = (int(v) for v in g["params"])
    for mode, tol in ((0, TOL["conv2d_tf32"]), (1, TOL["conv2d_3xtf32"])):
        for extra in ({}, {"epilogue": 1}, {"split_k": 3}, {"split_k": 1}):
            cfg = dict(extra, fp32_mode=mode)
            got = run_conv3d(B, g["x"], g["w"], g["b"], stride, pad, dil, groups, cfg=cfg, status=status)
            assert got.shape == g["y"].shape
            assert O.normalised_error(got, g["y"]) <= tol, cfg
    assert int(status.item()) == 0


# the reference's benchmark table (flextensor/configs/conv3d_config.py): 3-D ResNet-18 after the stem
@pytest.mark.parametrize("index", range(10))
def test_conv3d_reference_table(B, status, index):
    from flextensor_b200.configs.conv3d_config import conv3d_shapes
    n, c, d, h, w, k, _, ks, _, st, pad, dil, groups = conv3d_shapes[index]
    x, wt = _inputs(n, c, d, h, w, k, ks, ks, ks, groups, seed=300 + index)
    want = O.conv3d_ncdhw(x, wt, None, st, pad, dil, groups)
    for cfg, tol in ((None, TOL["conv2d_tf32"]), ({"fp32_mode": 1}, TOL["conv2d_3xtf32"])):
        got = run_conv3d(B, x, wt, None, st, pad, dil, groups, cfg=cfg, status=status)
        assert got.shape == want.shape
        assert O.normalised_error(got, want) <= tol, (index, cfg)
    assert int(status.item()) == 0


@pytest.mark.parametrize("cfg", [{}, {"cluster": 2}, {"cluster": 2, "split_k": 3}, {"tile_n": 32, "split_k": 1}, {"tile_h": 2},
                                 {"epilogue": 1}, {"epilogue": 1, "split_k": 2}, {"stages": 2}, {"relu": 1}])
@pytest.mark.parametrize("shape", [
    # n, c, d, h, w, k, (t, r, s), stride, padding, dilation, groups
    (2, 32, 5, 12, 16, 48, (3, 3, 3), (1, 1, 1), (1, 1, 1), (1, 1, 1), 1),
    (1, 40, 6, 9, 11, 20, (2, 3, 1), (2, 1, 2), (0, 1, 0), (1, 2, 1), 1),      # unaligned rows: per-thread stores
    (3, 24, 4, 8, 8, 36, (3, 1, 3), (1, 2, 1), (2, 0, 1), (2, 1, 1), 3),      # 8 channels per group
    (2, 10, 7, 6, 12, 15, (1, 3, 3), (3, 1, 1), (0, 1, 1), (1, 1, 1), 5),     # 2 channels per group, 3 filters per group
])
def test_conv3d_shapes_and_knobs(B, status, shape, cfg):
    n, c, d, h, w, k, taps, st, pad, dil, groups = shape
    x, wt = _inputs(n, c, d, h, w, k, *taps, groups, seed=310)
    bias = np.random.default_rng(311).standard_normal(k).astype(np.float32)
    want = O.conv3d_ncdhw(x, wt, bias, st, pad, dil, groups)
    if cfg.get("relu"):
        want = np.maximum(want, 0)
    try:
        got = run_conv3d(B, x, wt, bias, st, pad, dil, groups, cfg=cfg, status=status)
    except B.FtbError as exc:
        assert exc.code in (-2, -3), exc  # a knob set the shape cannot take is refused, never run wrong
        pytest.skip("refused: %s" % exc)
    assert got.shape == want.shape
    assert not np.isnan(got).any()
    assert O.normalised_error(got, want) <= TOL["conv2d_tf32"], (shape, cfg)
    assert int(status.item()) == 0


@pytest.mark.parametrize("cfg", [{"algo": 5}, {"algo": 5, "cluster": 1}, {"algo": 5, "cluster": 2}, {"algo": 5, "tile_h": 1},
                                 {"algo": 5, "epilogue": 1}, {"algo": 5, "relu": 1}, {}])
@pytest.mark.parametrize("shape", [
    # n, c, d, h, w, k, (t, r, s), padding, dilation  (stride 1)
    (2, 64, 8, 28, 28, 64, (3, 3, 3), (1, 1, 1), (1, 1, 1)),      # the first layer of the reference's table, batch 2
    (6, 32, 6, 16, 16, 48, (3, 3, 3), (1, 1, 1), (1, 1, 1)),      # enough tiles for the library to pick the slab kernel
    (3, 40, 2, 9, 12, 136, (3, 3, 3), (1, 1, 1), (1, 1, 1)),      # two input planes under three depth taps
    (2, 128, 1, 14, 14, 128, (3, 3, 3), (1, 1, 1), (1, 1, 1)),    # one input plane: two of three depth taps are padding
    (2, 24, 7, 10, 11, 20, (2, 3, 2), (1, 0, 1), (2, 1, 1)),      # depth dilation 2, rows that bulk stores cannot address
    (1, 96, 5, 12, 12, 72, (3, 1, 1), (0, 0, 0), (1, 1, 1)),      # depth taps only, no padding
])
def test_conv3d_on_the_slab_kernel(B, status, shape, cfg):
    """Stride-1 conv3d with one input slab per (depth tap, channel chunk) and the filter streamed (algo 5),
    single CTAs (which skip depth taps that fall into the padding) and CTA pairs (which load zeros there)."""
    n, c, d, h, w, k, taps, pad, dil = shape
    x, wt = _inputs(n, c, d, h, w, k, *taps, 1, seed=340)
    bias = np.random.default_rng(341).standard_normal(k).astype(np.float32)
    want = O.conv3d_ncdhw(x, wt, bias, 1, pad, dil, 1)
    if cfg.get("relu"):
        want = np.maximum(want, 0)
    try:
        got = run_conv3d(B, x, wt, bias, 1, pad, dil, 1, cfg=cfg, status=status, calls=2)
    except B.FtbError as exc:
        assert exc.code in (-2, -3), exc
        pytest.skip("refused: %s" % exc)
    assert got.shape == want.shape
    assert not np.isnan(got).any()
    assert O.normalised_error(got, want) <= TOL["conv2d_tf32"], (shape, cfg)
    assert int(status.item()) == 0


def test_conv3d_single_tap_is_the_batched_gemm(B, status):
    # 1x1x1, stride 1, no padding: a batched GEMM on the NCDHW tensors as they are
    x, wt = _inputs(2, 64, 4, 6, 8, 40, 1, 1, 1, 1, seed=320)
    want = O.conv3d_ncdhw(x, wt, None, 1, 0, 1, 1)
    before = B.lib().ftb_launch_count()
    got = run_conv3d(B, x, wt, None, 1, 0, 1, 1, cfg={"split_k": 1}, status=status)
    assert B.lib().ftb_launch_count() - before == 1  # no layout pass
    assert O.normalised_error(got, want) <= TOL["conv2d_tf32"]


def _random_cases(count, seed):
    rng = random.Random(seed)
    cases = []
    while len(cases) < count:
        groups = rng.choice([1, 1, 1, 2, 3])
        cg = rng.choice([1, 2, 3, 4, 6, 8, 16, 33, 40])
        kg = rng.choice([1, 3, 8, 16, 24, 40, 64])
        taps = tuple(rng.choice([1, 1, 2, 3, 3]) for _ in range(3))
        st = tuple(rng.choice([1, 1, 2, 3]) for _ in range(3))
        dil = tuple(rng.choice([1, 1, 2]) for _ in range(3))
        pad = tuple(rng.choice([0, 1, 1, 2]) for _ in range(3))
        dims = (rng.randint(1, 7), rng.randint(1, 14), rng.randint(1, 24))
        if any(O.out_size(dims[i], taps[i], st[i], pad[i], dil[i]) <= 0 for i in range(3)):
            continue
        n = rng.choice([1, 1, 2, 3])
        cfg = rng.choice([None, None, {"fp32_mode": 1}, {"split_k": 1}, {"cluster": 2}])
        cases.append((n, cg * groups, dims, kg * groups, taps, st, pad, dil, groups, rng.random() < 0.5, cfg))
    return cases


@pytest.mark.parametrize("case", _random_cases(40, 17))
def test_conv3d_random_shapes_against_the_oracle(B, status, case):
    n, c, dims, k, taps, st, pad, dil, groups, with_bias, cfg = case
    x, wt = _inputs(n, c, *dims, k, *taps, groups, seed=330)
    bias = np.random.default_rng(331).standard_normal(k).astype(np.float32) if with_bias else None
    want = O.conv3d_ncdhw(x, wt, bias, st, pad, dil, groups)
    got = run_conv3d(B, x, wt, bias, st, pad, dil, groups, cfg=cfg, status=status, calls=2)
    assert got.shape == want.shape
    tol = TOL["conv2d_3xtf32"] if (cfg or {}).get("fp32_mode") else TOL["conv2d_tf32"]
    assert O.normalised_error(got, want) <= tol, case
    assert int(status.item()) == 0


def test_conv3d_bad_arguments_are_refused(B):
    x = torch.zeros(1, 8, 4, 4, 4, device="cuda")
    w = torch.zeros(8, 8, 3, 3, 3, device="cuda")
    out = torch.zeros(1, 8, 2, 2, 2, device="cuda")
    with pytest.raises(ValueError):
        B.conv3d_ncdhw_f32(x, w, out, workspace=None)
    ws = torch.empty(B.conv3d_workspace_bytes(1, 8, 4, 4, 4, 8, 5, 5, 5, 1), dtype=torch.uint8, device="cuda")
    with pytest.raises(B.FtbError):   # a filter larger than the padded input
        B.conv3d_ncdhw_f32(x, torch.zeros(8, 8, 5, 5, 5, device="cuda"), out, workspace=ws)
    with pytest.raises(B.FtbError):   # the slab kernel takes conv3d at stride 1 only
        B.conv3d_ncdhw_f32(x, w, torch.zeros(1, 8, 1, 1, 1, device="cuda"), stride=2, workspace=ws, cfg={"algo": 5})
    with pytest.raises(ValueError):
        B.conv3d_ncdhw_f32(x, torch.zeros(8, 4, 3, 3, 3, device="cuda"), out, workspace=ws)


def test_conv3d_task_through_schedule_and_build(B):
    """The reference's flow for a conv3d task: schedule_with_config -> build -> func(*arrays), checked with
    the driver's own host comparison (optimize/common.py:test with check_result)."""
    from flextensor_b200.task import Task, register_task, conv3d
    from flextensor_b200.scheduler import schedule_with_config
    from flextensor_b200.runtime import build
    from flextensor_b200.utils import Config
    from flextensor_b200.measure import make_inputs
    from flextensor_b200.optimize.common import host_result
    task = Task("conv3d", "conv3d", conv3d, (2, 16, 4, 10, 12, 24, 3, 1, 1, 1, 1), "cuda", 0)
    register_task(task, override=True)
    s, bufs = schedule_with_config(task.key, Config([], {}))
    func = build(s, bufs, "cuda")
    arrays = make_inputs(bufs, torch.device("cuda", 0), low=-1.0, high=1.0)
    func(*arrays)
    before = B.lib().ftb_launch_count()
    func(*arrays)        # the second call finds the filter packed: layout pass (input only) + conv kernel
    func.check()
    assert B.lib().ftb_launch_count() - before == 2
    ops, bufs2 = task.func(*task.args)
    want = host_result(ops, bufs2, arrays)
    got = arrays[-1].double().cpu().numpy()
    assert O.normalised_error(got, want) <= TOL["conv2d_tf32"]
