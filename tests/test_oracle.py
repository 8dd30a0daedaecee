"""The oracle (oracle/) against the committed golden vectors, against torch CPU on the very
cases the reference's own tests use, and its numpy and C forms against each other."""
import os

import numpy as np
import pytest
import torch

from conftest import GOLDEN_DIR
from oracle import ft_oracle as O


def _load(name):
    return np.load(os.path.join(GOLDEN_DIR, name + ".npz"))


def test_golden_conv2d_grouped():
    g = _load("conv2d_grouped")
    stride, pad, dil, groups = (int(v) for v in g["params"])
    y = O.conv2d_nchw(g["x"], g["w"], g["b"], stride, pad, dil, groups)
    assert O.normalised_error(y, g["y"]) < 1e-6


def test_golden_conv2d_3x3():
    g = _load("conv2d_3x3")
    assert O.normalised_error(O.conv2d_nchw(g["x"], g["w"], None, 1, 1, 1, 1), g["y"]) < 1e-6


def test_golden_depthwise():
    g = _load("depthwise_f3")
    stride, pad, dil = (int(v) for v in g["params"])
    assert O.normalised_error(O.depthwise_conv2d_nchw(g["x"], g["w"], g["b"], stride, pad, dil), g["y"]) < 1e-6


def test_golden_gemms():
    g = _load("gemm_f32")
    assert O.normalised_error(O.gemm(g["a"], g["b"]), g["y"]) < 1e-6
    g = _load("bgemm_bf16")
    y = O.batch_gemm(O.from_bf16_bits(g["a_bits"]), O.from_bf16_bits(g["b_bits"]))
    assert O.normalised_error(y, g["y"]) < 1e-6
    g = _load("gemm_int8")
    assert (O.gemm_int8(g["a"], g["b"]) == g["y"]).all()


def test_conv2d_as_reference_test_does():
    """flextensor/test/test_ops.py:85-115: groups 3, stride 2, padding 1, dilation 2, bias, inputs x1000,
    compared with torch at rtol 1e-5*1000."""
    rng = np.random.default_rng(7)
    x = (rng.uniform(-1, 1, (4, 6, 7, 7)) * 1000).astype(np.float32)
    w = (rng.uniform(-1, 1, (9, 2, 3, 3)) * 1000).astype(np.float32)
    b = (rng.uniform(-1, 1, 9) * 1000).astype(np.float32)
    want = torch.nn.functional.conv2d(torch.tensor(x), torch.tensor(w), torch.tensor(b), stride=2, padding=1,
                                      dilation=2, groups=3).numpy()
    got = O.conv2d_nchw(x, w, b, stride=2, padding=1, dilation=2, groups=3)
    np.testing.assert_allclose(got, want, rtol=1e-5 * 1000)


def test_golden_conv3d_grouped():
    g = _load("conv3d_grouped")
    stride, pad, dil, groups = (int(v) for v in g["params"])
    y = O.conv3d_ncdhw(g["x"], g["w"], g["b"], stride, pad, dil, groups)
    assert O.normalised_error(y, g["y"]) < 1e-6


def test_conv3d_as_reference_test_does():
    """flextensor/test/test_ops.py:187-214: [4,6,7,7,7] input x100, [9,2,3,3,3] filter x100, bias x100, stride 2,
    padding 1, dilation 2, groups 3, compared with torch at rtol 1e-5; then per-axis parameters."""
    rng = np.random.default_rng(9)
    x = (rng.random((4, 6, 7, 7, 7)) * 100).astype(np.float32)
    w = (rng.random((9, 2, 3, 3, 3)) * 100).astype(np.float32)
    b = (rng.random(9) * 100).astype(np.float32)
    want = torch.nn.functional.conv3d(torch.tensor(x).double(), torch.tensor(w).double(), torch.tensor(b).double(),
                                      stride=2, padding=1, dilation=2, groups=3).numpy()
    got = O.conv3d_ncdhw(x, w, b, stride=2, padding=1, dilation=2, groups=3)
    np.testing.assert_allclose(got, want, rtol=1e-5)
    x = rng.standard_normal((2, 8, 5, 9, 6)).astype(np.float32)
    w = rng.standard_normal((6, 4, 2, 3, 1)).astype(np.float32)
    want = torch.nn.functional.conv3d(torch.tensor(x).double(), torch.tensor(w).double(), None, stride=(1, 2, 3),
                                      padding=(1, 0, 2), dilation=(2, 1, 1), groups=2).numpy()
    got = O.conv3d_ncdhw(x, w, None, stride=(1, 2, 3), padding=(1, 0, 2), dilation=(2, 1, 1), groups=2)
    assert got.shape == want.shape
    assert O.normalised_error(got, want) < 1e-6


def test_depthwise_as_reference_test_does():
    """flextensor/test/test_ops.py:152-184: weight [18,1,3,3] for torch is [6,3,3,3] for the op; rtol 1e-5."""
    rng = np.random.default_rng(8)
    x = (rng.random((4, 6, 7, 7)) * 100).astype(np.float32)
    w = (rng.random((18, 1, 3, 3)) * 100).astype(np.float32)
    b = (rng.random(18) * 100).astype(np.float32)
    want = torch.nn.functional.conv2d(torch.tensor(x), torch.tensor(w), torch.tensor(b), stride=2, padding=1,
                                      dilation=2, groups=6).numpy()
    got = O.depthwise_conv2d_nchw(x, w.reshape(6, 3, 3, 3), b, stride=2, padding=1, dilation=2)
    np.testing.assert_allclose(got, want, rtol=1e-5)


@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False), (True, True)])
def test_gemm_variants_against_torch(ta, tb):
    a, b = O.gemm_inputs(19, 23, 31, seed=5)
    want = (torch.tensor(a).double() @ torch.tensor(b).double()).numpy()
    got = O.gemm(a.T.copy() if ta else a, b.T.copy() if tb else b, ta, tb, out_dtype=np.float64)
    np.testing.assert_allclose(got, want, rtol=1e-12)


def test_zero_pad2d_forms():
    x = np.arange(2 * 3 * 4 * 5, dtype=np.float32).reshape(2, 3, 4, 5)
    assert O.zero_pad2d(x, 0).shape == x.shape
    p = O.zero_pad2d(x, (1, 2))
    assert p.shape == (2, 3, 6, 9) and p[0, 0, 0].sum() == 0 and (p[:, :, 1:5, 2:7] == x).all()
    p = O.zero_pad2d(x, (1, 0, 2, 3))
    assert p.shape == (2, 3, 5, 10) and (p[:, :, 1:, 2:7] == x).all()


def test_bf16_rounding_matches_torch():
    x = np.random.default_rng(3).standard_normal(4096).astype(np.float32) * 3
    want = torch.tensor(x).bfloat16().float().numpy()
    assert (O.round_to_bf16(x) == want).all()


def test_int8_routes_agree():
    a, b = O.gemm_int8_inputs(40, 24, 300, seed=9)
    assert (O.gemm_int8(a, b) == O.gemm_int8_direct(a, b)).all()
    assert (O.gemm_int8(a, b.T.copy(), transposeB=True) == O.gemm_int8_direct(a, b)).all()
    extreme = np.full((4, 8192), 127, dtype=np.int8)
    assert (O.gemm_int8(extreme, extreme.T.copy()) == 127 * 127 * 8192).all()  # largest magnitude fits int32


def test_c_restatement_agrees(c_oracle):
    a, b = O.gemm_inputs(21, 17, 45, seed=11)
    assert O.normalised_error(c_oracle.gemm_f32_naive(a, b), O.gemm(a, b)) < 1e-6
    assert O.normalised_error(c_oracle.gemm_f32_naive(a.T.copy(), b, ta=True), O.gemm(a, b)) < 1e-6
    assert O.normalised_error(c_oracle.gemm_f32_tiled(a, b, 8, 64, 16), O.gemm(a, b)) < 1e-5
    a8, b8 = O.gemm_int8_inputs(13, 29, 70, seed=12)
    assert (c_oracle.gemm_s8_naive(a8, b8) == O.gemm_int8(a8, b8)).all()
    assert (c_oracle.gemm_s8_tiled(a8, b8) == O.gemm_int8(a8, b8)).all()
    x, w = O.conv2d_inputs(2, 6, 9, 11, 8, 3, 3, groups=2, seed=13)
    got = c_oracle.conv2d_naive(x, w, None, (2, 1), (1, 2), (1, 2), 2)
    assert O.normalised_error(got, O.conv2d_nchw(x, w, None, (2, 1), (1, 2), (1, 2), 2)) < 1e-6
    x, w = O.conv2d_inputs(1, 5, 10, 12, 7, 3, 3, seed=14)
    assert O.normalised_error(c_oracle.conv2d_tiled(x, w, (1, 1), (1, 1), (1, 1), 4),
                              O.conv2d_nchw(x, w, None, 1, 1, 1)) < 1e-5
    assert O.normalised_error(c_oracle.conv2d_tiled(x, w, (2, 2), (2, 2), (2, 2), 3),
                              O.conv2d_nchw(x, w, None, 2, 2, 2)) < 1e-5
    x, w = O.depthwise_inputs(2, 5, 9, 10, 2, 3, 3, seed=15)
    assert O.normalised_error(c_oracle.dwconv2d_naive(x, w, None, (1, 1), (1, 1), (1, 1)),
                              O.depthwise_conv2d_nchw(x, w, None, 1, 1, 1)) < 1e-6
    assert O.normalised_error(c_oracle.dwconv2d_tiled(x, w, (2, 2), (1, 1), (1, 1), 2),
                              O.depthwise_conv2d_nchw(x, w, None, 2, 1, 1)) < 1e-5
    items = [O.batch_gemm_item(i, 10, 12, 20) for i in range(2)]
    a = np.stack([i[0] for i in items])
    b = np.stack([i[1] for i in items])
    got = O.from_bf16_bits(c_oracle.bgemm_bf16_tiled(O.to_bf16_bits(a), O.to_bf16_bits(b)))
    assert O.bf16_output_ok(got, O.batch_gemm(a, b))


def test_batch_items_do_not_depend_on_shard_count():
    a0, _ = O.batch_gemm_item(5, 8, 8, 8)
    a1, _ = O.batch_gemm_item(5, 8, 8, 8)
    a2, _ = O.batch_gemm_item(6, 8, 8, 8)
    assert (a0 == a1).all() and not (a0 == a2).all()


def test_conv1d_and_packed_1x1_restatements_against_torch():
    """conv1d with groups, stride and dilation against torch CPU (the comparator the reference's op
    tests use); the packed 1x1 form against a literal loop nest."""
    import torch
    rng = np.random.default_rng(7)
    x = rng.standard_normal((2, 6, 31)).astype(np.float32)
    w = rng.standard_normal((9, 2, 4)).astype(np.float32)
    b = rng.standard_normal(9).astype(np.float32)
    got = O.conv1d(x, w, b, stride=2, padding=3, dilation=2, groups=3)
    want = torch.nn.functional.conv1d(torch.tensor(x), torch.tensor(w), torch.tensor(b), stride=2, padding=3,
                                      dilation=2, groups=3).numpy()
    assert got.shape == want.shape and O.normalised_error(got, want) < 1e-5
    a = rng.standard_normal((2, 5, 7)).astype(np.float32)
    m = rng.standard_normal((3, 5)).astype(np.float32)
    loops = np.zeros((2, 3, 7))
    for bi in range(2):
        for k in range(3):
            for i in range(7):
                loops[bi, k, i] = sum(float(a[bi, rc, i]) * float(m[k, rc]) for rc in range(5))
    assert O.normalised_error(O.conv2d_1x1_packed(a, m), loops) < 1e-6
