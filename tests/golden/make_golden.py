"""Generates the golden fixtures of this directory: ``python tests/golden/make_golden.py``.

The reference (pku-liang/FlexTensor) holds no golden vectors for these operators and cannot
run here (it needs an un-vendored TVM fork), so the vectors come from the numpy
restatement in ``oracle/ft_oracle.py`` on seeded inputs, each cross-checked at generation
time against torch CPU - the comparator the reference's own tests use
(flextensor/test/test_ops.py:85-115,152-184) - and against the plain-C restatement.
A fixture stores only the seed-independent facts a test needs: shapes/parameters, the
input arrays (small) and the expected output.
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import ft_oracle as O  # noqa: E402
from oracle import c_oracle as CO  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def save(name, **arrays):
    path = os.path.join(HERE, name + ".npz")
    np.savez_compressed(path, **arrays)
    print("wrote", path, os.path.getsize(path), "bytes")


def main():
    # conv2d: groups, stride, dilation, bias - the reference's test case shape
    rng = np.random.Generator(np.random.PCG64(100))
    x = rng.uniform(-1, 1, (4, 6, 7, 7)).astype(np.float32)
    w = rng.uniform(-1, 1, (9, 2, 3, 3)).astype(np.float32)
    b = rng.uniform(-1, 1, 9).astype(np.float32)
    y = O.conv2d_nchw(x, w, b, stride=2, padding=1, dilation=2, groups=3)
    t = torch.nn.functional.conv2d(torch.tensor(x), torch.tensor(w), torch.tensor(b), stride=2, padding=1,
                                   dilation=2, groups=3).numpy()
    assert O.normalised_error(t, y) < 1e-5
    assert O.normalised_error(CO.conv2d_naive(x, w, b, (2, 2), (1, 1), (2, 2), 3), y) < 1e-6
    save("conv2d_grouped", x=x, w=w, b=b, y=y, params=np.array([2, 1, 2, 3]))

    # conv3d: the reference's test case shape (flextensor/test/test_ops.py:187-214): 6 channels in 3 groups,
    # 9 filters of 3x3x3, stride 2, padding 1, dilation 2, bias
    rng = np.random.Generator(np.random.PCG64(106))
    x = rng.uniform(-1, 1, (4, 6, 7, 7, 7)).astype(np.float32)
    w = rng.uniform(-1, 1, (9, 2, 3, 3, 3)).astype(np.float32)
    b = rng.uniform(-1, 1, 9).astype(np.float32)
    y = O.conv3d_ncdhw(x, w, b, stride=2, padding=1, dilation=2, groups=3)
    t = torch.nn.functional.conv3d(torch.tensor(x), torch.tensor(w), torch.tensor(b), stride=2, padding=1,
                                   dilation=2, groups=3).numpy()
    assert O.normalised_error(t, y) < 1e-5
    save("conv3d_grouped", x=x, w=w, b=b, y=y, params=np.array([2, 1, 2, 3]))

    # conv2d: a 3x3 stride-1 pad-1 layer with a channel count that is not a multiple of 32
    x, w = O.conv2d_inputs(2, 20, 12, 14, 24, 3, 3, seed=101)
    y = O.conv2d_nchw(x, w, None, 1, 1, 1, 1)
    t = torch.nn.functional.conv2d(torch.tensor(x), torch.tensor(w), None, 1, 1).numpy()
    assert O.normalised_error(t, y) < 1e-5
    save("conv2d_3x3", x=x, w=w, y=y, params=np.array([1, 1, 1, 1]))

    # depthwise: factor 3, stride 2, dilation 2, bias - the reference's test case shape
    rng = np.random.Generator(np.random.PCG64(102))
    x = rng.random((4, 6, 7, 7)).astype(np.float32)
    w = rng.random((6, 3, 3, 3)).astype(np.float32)
    b = rng.random(18).astype(np.float32)
    y = O.depthwise_conv2d_nchw(x, w, b, stride=2, padding=1, dilation=2)
    t = torch.nn.functional.conv2d(torch.tensor(x), torch.tensor(w.reshape(18, 1, 3, 3)), torch.tensor(b), stride=2,
                                   padding=1, dilation=2, groups=6).numpy()
    assert O.normalised_error(t, y) < 1e-5
    assert O.normalised_error(CO.dwconv2d_naive(x, w, b, (2, 2), (1, 1), (2, 2)), y) < 1e-6
    save("depthwise_f3", x=x, w=w, b=b, y=y, params=np.array([2, 1, 2]))

    # gemm fp32, ragged sizes (multiples of 4 so that rows stay 16-byte aligned)
    a, bm = O.gemm_inputs(72, 40, 100, seed=103)
    y = O.gemm(a, bm)
    assert O.normalised_error(CO.gemm_f32_naive(a, bm), y) < 1e-6
    assert O.normalised_error((torch.tensor(a).double() @ torch.tensor(bm).double()).float().numpy(), y) < 1e-6
    save("gemm_f32", a=a, b=bm, y=y)

    # batched gemm bf16 (values stored as float32 that are exactly bf16)
    items = [O.batch_gemm_item(i, 40, 48, 72, seed=104) for i in range(3)]
    a = np.stack([it[0] for it in items])
    bm = np.stack([it[1] for it in items])
    y = O.batch_gemm(a, bm)
    c_bits = CO.bgemm_bf16_naive(O.to_bf16_bits(a), O.to_bf16_bits(bm), out_f32=True)
    assert O.normalised_error(c_bits, y) < 1e-6
    save("bgemm_bf16", a_bits=O.to_bf16_bits(a), b_bits=O.to_bf16_bits(bm), y=y)

    # int8 gemm
    a, bm = O.gemm_int8_inputs(48, 64, 144, seed=105)
    y = O.gemm_int8(a, bm)
    assert (y == O.gemm_int8_direct(a, bm)).all() and (y == CO.gemm_s8_naive(a, bm)).all()
    save("gemm_int8", a=a, b=bm, y=y)


if __name__ == "__main__":
    main()
