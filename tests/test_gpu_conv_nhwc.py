"""conv2d on channels-last tensors (the layout rewrite of a conv2d task): the same kernels reading [N,H,W,C]
in place and writing [N,P,Q,K], through the C ABI and through ``schedule_with_config(..., rewrite=True)``,
against the numpy oracle of the NCHW op on the transposed tensors.

Tolerances are those of conv2d: normalised error <= 5e-3 single-pass TF32, <= 1e-4 3xTF32.
"""
import random

import numpy as np
import pytest
import torch

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


def run_nhwc(B, x_nchw, w, bias=None, stride=1, padding=0, dilation=1, groups=1, cfg=None, status=None, calls=1):
    """Runs the channels-last entry on the NHWC form of ``x_nchw``; returns the result back in NCHW order."""
    n, c, h, wd = x_nchw.shape
    k, _, r, s = w.shape
    p = O.out_size(h, r, stride, padding, dilation)
    q = O.out_size(wd, s, stride, padding, dilation)
    x = torch.from_numpy(np.ascontiguousarray(x_nchw.transpose(0, 2, 3, 1))).cuda()
    wt = torch.from_numpy(w).cuda()
    bt = torch.from_numpy(bias).cuda() if bias is not None else None
    out = torch.full((n, p, q, k), float("nan"), device="cuda")
    ws = torch.empty(B.conv2d_nhwc_workspace_bytes(c, k, r, s, groups), dtype=torch.uint8, device="cuda")
    for i in range(calls):
        if i:
            out.fill_(float("nan"))
        B.conv2d_nhwc_f32(x, wt, out, bt, (stride, stride), (padding, padding), (dilation, dilation), groups, cfg=cfg,
                          workspace=ws, status=status, prepacked=i > 0)
    torch.cuda.synchronize()
    return out.cpu().numpy().transpose(0, 3, 1, 2)


@pytest.mark.parametrize("cfg", [{}, {"algo": 1}, {"algo": 2}, {"algo": 2, "cluster": 2}, {"algo": 1, "cluster": 2},
                                 {"algo": 1, "split_k": 3}, {"algo": 2, "split_k": 3}, {"epilogue": 1}, {"relu": 1},
                                 {"fp32_mode": 1}, {"algo": 1, "tile_n": 32, "split_k": 1}])
@pytest.mark.parametrize("shape", [
    # n, c, h, w, k, r, stride, pad, dil, groups
    (2, 64, 56, 56, 64, 3, 1, 1, 1, 1),      # the ResNet stage-2 layer
    (3, 32, 20, 24, 48, 3, 1, 1, 1, 1),
    (1, 40, 9, 11, 20, 3, 1, 1, 1, 1),       # 11 output columns: no 16-byte rows in NCHW, fine channels-last
    (2, 64, 14, 14, 128, 1, 1, 0, 1, 1),     # 1x1
    (2, 32, 29, 31, 64, 3, 2, 2, 2, 1),      # stride 2, dilation 2
    (5, 16, 7, 7, 24, 3, 1, 1, 1, 1),        # several images per tile
    (2, 24, 14, 14, 36, 3, 1, 1, 1, 3),      # 8 channels in, 12 out per group
    (1, 64, 28, 28, 64, 1, 2, 0, 1, 1),      # strided 1x1
])
def test_conv2d_nhwc_shapes_and_knobs(B, status, shape, cfg):
    n, c, h, w, k, r, stride, pad, dil, groups = shape
    x, wt = O.conv2d_inputs(n, c, h, w, k, r, r, groups=groups, seed=400)
    bias = np.random.default_rng(401).standard_normal(k).astype(np.float32)
    want = O.conv2d_nchw(x, wt, bias, stride, pad, dil, groups)
    if cfg.get("relu"):
        want = np.maximum(want, 0)
    try:
        got = run_nhwc(B, x, wt, bias, stride, pad, dil, groups, cfg=cfg, status=status)
    except B.FtbError as exc:
        assert exc.code in (-2, -3), exc  # a knob set the shape cannot take is refused, never run wrong
        pytest.skip("refused: %s" % exc)
    assert got.shape == want.shape
    assert not np.isnan(got).any()
    tol = TOL["conv2d_3xtf32"] if cfg.get("fp32_mode") else TOL["conv2d_tf32"]
    assert O.normalised_error(got, want) <= tol, (shape, cfg)
    assert int(status.item()) == 0


def _random_cases(count, seed):
    rng = random.Random(seed)
    cases = []
    while len(cases) < count:
        groups = rng.choice([1, 1, 1, 2, 4])
        cg = rng.choice([4, 8, 12, 16, 32, 40, 64])
        kg = rng.choice([4, 8, 16, 24, 32, 48, 64, 100, 128])
        r = rng.choice([1, 1, 2, 3, 3, 3, 5])
        stride, dil, pad = rng.choice([1, 1, 1, 2, 3]), rng.choice([1, 1, 1, 2]), rng.choice([0, 0, 1, 1, 2])
        h = rng.randint(max(1, dil * (r - 1) + 1 - 2 * pad), 24)
        w = rng.randint(max(1, dil * (r - 1) + 1 - 2 * pad), 40)
        n = rng.choice([1, 1, 2, 3, 5, 9])
        if O.out_size(h, r, stride, pad, dil) <= 0 or O.out_size(w, r, stride, pad, dil) <= 0:
            continue
        cfg = rng.choice([None, None, {"fp32_mode": 1}, {"algo": 1}, {"split_k": 1}])
        cases.append((n, cg * groups, h, w, kg * groups, r, stride, pad, dil, groups, rng.random() < 0.5, cfg))
    return cases


@pytest.mark.parametrize("case", _random_cases(40, 19))
def test_conv2d_nhwc_random_shapes_against_the_oracle(B, status, case):
    n, c, h, w, k, r, stride, pad, dil, groups, with_bias, cfg = case
    x, wt = O.conv2d_inputs(n, c, h, w, k, r, r, groups=groups, seed=410)
    bias = np.random.default_rng(411).standard_normal(k).astype(np.float32) if with_bias else None
    want = O.conv2d_nchw(x, wt, bias, stride, pad, dil, groups)
    got = run_nhwc(B, x, wt, bias, stride, pad, dil, groups, cfg=cfg, status=status, calls=2)  # second call: prepacked
    assert got.shape == want.shape
    tol = TOL["conv2d_3xtf32"] if (cfg or {}).get("fp32_mode") else TOL["conv2d_tf32"]
    assert O.normalised_error(got, want) <= tol, case
    assert int(status.item()) == 0


def test_conv2d_nhwc_launches_no_layout_pass_once_the_filter_is_packed(B, status):
    x, wt = O.conv2d_inputs(4, 64, 56, 56, 64, 3, 3, seed=420)
    xt = torch.from_numpy(np.ascontiguousarray(x.transpose(0, 2, 3, 1))).cuda()
    w = torch.from_numpy(wt).cuda()
    out = torch.empty(4, 56, 56, 64, device="cuda")
    ws = torch.empty(B.conv2d_nhwc_workspace_bytes(64, 64, 3, 3, 1), dtype=torch.uint8, device="cuda")
    B.conv2d_nhwc_f32(xt, w, out, None, (1, 1), (1, 1), (1, 1), 1, workspace=ws, status=status)
    first = out.clone()
    before = B.lib().ftb_launch_count()
    B.conv2d_nhwc_f32(xt, w, out, None, (1, 1), (1, 1), (1, 1), 1, workspace=ws, status=status, prepacked=True)
    torch.cuda.synchronize()
    assert B.lib().ftb_launch_count() - before == 1
    assert torch.equal(first, out)
    want = O.conv2d_nchw(x, wt, None, 1, 1, 1, 1)
    assert O.normalised_error(out.cpu().numpy().transpose(0, 3, 1, 2), want) <= TOL["conv2d_tf32"]


def test_conv2d_nhwc_refuses_what_it_cannot_address(B):
    ws = torch.empty(1 << 20, dtype=torch.uint8, device="cuda")
    x = torch.zeros(1, 8, 8, 6, device="cuda")           # 6 channels: rows of 24 bytes
    w = torch.zeros(8, 6, 3, 3, device="cuda")
    out = torch.zeros(1, 6, 6, 8, device="cuda")
    with pytest.raises(B.FtbError) as err:
        B.conv2d_nhwc_f32(x, w, out, workspace=ws)
    assert err.value.code == -2
    x = torch.zeros(1, 8, 8, 8, device="cuda")
    w = torch.zeros(6, 8, 3, 3, device="cuda")           # 6 output channels
    out = torch.zeros(1, 6, 6, 6, device="cuda")
    with pytest.raises(B.FtbError) as err:
        B.conv2d_nhwc_f32(x, w, out, workspace=ws)
    assert err.value.code == -2
    with pytest.raises(ValueError):
        B.conv2d_nhwc_f32(x, torch.zeros(8, 8, 3, 3, device="cuda"), torch.zeros(1, 6, 6, 8, device="cuda"),
                          workspace=None)


def test_rewritten_task_through_schedule_and_build(B):
    """schedule_with_config(task_key, configs, rewrite=True): the conv2d task planned on channels-last buffers,
    built and run like any other plan, checked with the drivers' host comparison."""
    from flextensor_b200.scheduler import schedule_with_config
    from flextensor_b200.runtime import build
    from flextensor_b200.utils import Config
    from flextensor_b200.measure import make_inputs
    from flextensor_b200.optimize.common import host_result
    from flextensor_b200.task import TASK_TABLE
    key = "conv2d_res_b13_(1, 64, 56, 56, 64, 3, 1, 1, 1, 1)_cuda(0)"
    s, bufs = schedule_with_config(key, Config([], None), rewrite=True)
    assert [tuple(int(v) for v in b.shape) for b in bufs] == [(1, 56, 56, 64), (64, 64, 3, 3), (1, 56, 56, 64)]
    func = build(s, bufs, "cuda")
    arrays = make_inputs(bufs, torch.device("cuda", 0), low=-1.0, high=1.0)
    func(*arrays)
    first = arrays[-1].clone()
    func(*arrays)        # second call: the filter is found packed
    func.check()
    # (a batch-1 layer splits its taps over CTAs whose partial sums are added in any order)
    assert torch.allclose(first, arrays[-1], rtol=1e-5, atol=1e-4)
    twin = TASK_TABLE["conv2d_res_b13-nhwc_(1, 64, 56, 56, 64, 3, 1, 1, 1, 1)_cuda(0)"]
    ops, bufs2 = twin.func(*twin.args)
    want = host_result(ops, bufs2, arrays)
    assert O.normalised_error(arrays[-1].double().cpu().numpy(), want) <= TOL["conv2d_tf32"]
