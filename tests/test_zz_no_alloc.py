"""The allocation-free conv2d entry point (collected last on purpose: a run that stops at the
first failure has by then run every other test).

Some users of the library cannot allocate device memory - they get their buffers from another
runtime, or run where allocation is forbidden once serving has started - so they cannot hand
the regular conv2d its workspace.  ``ftb_conv2d_nchw_f32_noalloc`` keeps a fixed 8 MiB
workspace inside the library instead.  Here it is called through the C ABI twice in a row, on
two different shapes, and each result is compared with the regular entry point's.  The two
paths run the same kernels with the same knobs (no K split, so no atomics), so the outputs must
be bit-identical; the
second call also shows that what the first one left in the shared workspace does no harm.
"""
import numpy as np
import pytest
import torch

from oracle import ft_oracle as O

pytestmark = pytest.mark.gpu


def _both(B, x, w, bias, stride, pad, dil, groups, status, cfg=None):
    cfg = {"fp32_mode": 1, "split_k": 1} if cfg is None else cfg
    n, c, h, wd = x.shape
    k, _, r, s = w.shape
    p = O.out_size(h, r, stride, pad, dil)
    q = O.out_size(wd, s, stride, pad, dil)
    xd, wdv = torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda()
    bd = torch.from_numpy(bias).cuda() if bias is not None else None
    args = (bd, (stride, stride), (pad, pad), (dil, dil), groups)
    ref = torch.full((n, k, p, q), float("nan"), device="cuda")
    ws = torch.empty(B.conv2d_workspace_bytes(n, c, h, wd, k, r, s, groups), dtype=torch.uint8, device="cuda")
    B.conv2d_nchw_f32(xd, wdv, ref, *args, cfg=cfg, workspace=ws, status=status)
    got = torch.full((n, k, p, q), float("nan"), device="cuda")
    torch.cuda.synchronize()
    allocated = torch.cuda.memory_allocated()
    B.conv2d_nchw_f32_noalloc(xd, wdv, got, *args, cfg=cfg, status=status)
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == allocated     # torch's allocator was not touched either
    return got.cpu().numpy(), ref.cpu().numpy()


def test_noalloc_conv_matches_regular_entry_point_twice(native_lib):
    from flextensor_b200 import backend as B
    assert B.lib().ftb_device_check() == 0
    status = B.new_status()
    # first call: ResNet-50 stage-2 layer (workspace 1.4 MB)
    x, w = O.conv2d_inputs(1, 64, 56, 56, 64, 3, 3, seed=1)
    got, ref = _both(B, x, w, None, 1, 1, 1, 1, status)
    assert np.array_equal(got, ref)
    assert O.normalised_error(got, O.conv2d_nchw(x, w, None, 1, 1, 1)) <= O.TOLERANCE["conv2d_3xtf32"]
    # second call straight after, another shape (stride, dilation, bias, groups): stale scratch is harmless
    x, w = O.conv2d_inputs(2, 24, 17, 19, 36, 3, 3, groups=3, seed=2)
    bias = np.linspace(-2, 2, 36).astype(np.float32)
    got, ref = _both(B, x, w, bias, 2, 2, 2, 3, status)
    assert np.array_equal(got, ref)
    assert O.normalised_error(got, O.conv2d_nchw(x, w, bias, 2, 2, 2, 3)) <= O.TOLERANCE["conv2d_3xtf32"]
    B.check_status(status)


def test_noalloc_conv_every_workspace_layout_back_to_back(native_lib):
    """The shared array is laid out differently by each lowering of the conv: a channels-last copy
    (per-tap and slab kernels), one row of taps x channels per output pixel (few input channels),
    only the pixels a strided 1x1 filter reads, groups padded to four channels.  Each case runs
    straight after one that left another layout behind and must still agree with the regular
    entry point: bit for bit where the kernels add nothing in global memory, within the conv
    tolerance where the library's default splits the reduction over CTAs."""
    from flextensor_b200 import backend as B
    status = B.new_status()
    cases = [
        # (n, c, h, w, k, r, stride, pad, groups, cfg, exact)
        (1, 3, 64, 64, 16, 7, 2, 3, 1, {"algo": 4, "split_k": 1}, True),      # im2col rows
        (2, 32, 28, 28, 48, 3, 1, 1, 1, {"algo": 2, "split_k": 1}, True),     # slab kernel, default TF32
        (2, 64, 28, 28, 32, 1, 2, 0, 1, {"algo": 1, "split_k": 1}, True),     # strided 1x1: kept pixels only
        (1, 64, 56, 56, 64, 3, 1, 1, 1, {}, False),                           # library defaults: split reduction
        (2, 18, 15, 13, 12, 3, 1, 1, 6, {"split_k": 1}, True),                # 3 channels per group, padded to 4
        (1, 3, 64, 64, 16, 7, 2, 3, 1, {"algo": 4, "split_k": 1}, True),      # and the first layout again
    ]
    for n, c, h, w, k, r, stride, pad, groups, cfg, exact in cases:
        x, wt = O.conv2d_inputs(n, c, h, w, k, r, r, groups=groups, seed=5)
        got, ref = _both(B, x, wt, None, stride, pad, 1, groups, status, cfg=cfg)
        if exact:
            assert np.array_equal(got, ref), (n, c, h, w, k, r, stride, pad, groups, cfg)
        else:
            assert O.normalised_error(got, ref) <= O.TOLERANCE["conv2d_tf32"]
        assert O.normalised_error(got, O.conv2d_nchw(x, wt, None, stride, pad, 1, groups)) <= O.TOLERANCE["conv2d_tf32"]
    B.check_status(status)


def test_noalloc_conv_refuses_oversized_shapes(native_lib):
    from flextensor_b200 import backend as B
    n, c, h, w, k = 8, 64, 112, 112, 64        # 25.7 MB channels-last copy alone
    assert B.conv2d_workspace_bytes(n, c, h, w, k, 3, 3, 1) > B.NOALLOC_SCRATCH_BYTES
    x = torch.zeros(n, c, h, w, device="cuda")
    wt = torch.zeros(k, c, 3, 3, device="cuda")
    out = torch.zeros(n, k, h, w, device="cuda")
    with pytest.raises(B.FtbError) as err:
        B.conv2d_nchw_f32_noalloc(x, wt, out, padding=(1, 1))
    assert err.value.code == -7
