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


def _both(B, x, w, bias, stride, pad, dil, groups, status):
    n, c, h, wd = x.shape
    k, _, r, s = w.shape
    p = O.out_size(h, r, stride, pad, dil)
    q = O.out_size(wd, s, stride, pad, dil)
    xd, wdv = torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda()
    bd = torch.from_numpy(bias).cuda() if bias is not None else None
    args = (bd, (stride, stride), (pad, pad), (dil, dil), groups)
    ref = torch.full((n, k, p, q), float("nan"), device="cuda")
    ws = torch.empty(B.conv2d_workspace_bytes(n, c, h, wd, k, r, s, groups), dtype=torch.uint8, device="cuda")
    B.conv2d_nchw_f32(xd, wdv, ref, *args, cfg={"fp32_mode": 1, "split_k": 1}, workspace=ws, status=status)
    got = torch.full((n, k, p, q), float("nan"), device="cuda")
    torch.cuda.synchronize()
    allocated = torch.cuda.memory_allocated()
    B.conv2d_nchw_f32_noalloc(xd, wdv, got, *args, cfg={"fp32_mode": 1, "split_k": 1}, status=status)
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
