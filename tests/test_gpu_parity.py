"""Parity of the sm_100a kernels, called through the C ABI, against the oracle.

Tolerances (stated once in oracle/ft_oracle.py:TOLERANCE):
  int8 GEMM                     bit-exact
  GEMM fp32, 3xTF32             normalised error <= 1e-4   (|x-y| / max(|y|, rms(y)))
  GEMM fp32, single-pass TF32   normalised error <= 5e-3   (reported mode, not the default)
  conv2d TF32 / 3xTF32          5e-3 / 1e-4
  depthwise fp32                1e-5
  batched GEMM bf16             |x-y| <= 2^-7 |y| + 2^-8 rms(y) for bf16 output; 1e-5 for fp32 output
"""
import os

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
    B.check_status(st)  # no kernel may have given up a wait


def _load(name):
    return np.load(os.path.join(GOLDEN_DIR, name + ".npz"))


def dev(x):
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


def bf16_dev(values_f32):
    return dev(values_f32).to(torch.bfloat16)


# ---------------------------------------------------------------- GEMM fp32
def run_gemm_f32(B, a, b, ta=False, tb=False, cfg=None, status=None):
    m = a.shape[1] if ta else a.shape[0]
    n = b.shape[0] if tb else b.shape[1]
    c = torch.full((m, n), float("nan"), device="cuda")
    B.gemm_f32(dev(a), dev(b), c, ta, tb, cfg=cfg, status=status)
    torch.cuda.synchronize()
    return c.cpu().numpy()


def test_gemm_f32_golden(B, status):
    g = _load("gemm_f32")
    got = run_gemm_f32(B, g["a"], g["b"], cfg={"fp32_mode": 1}, status=status)
    assert O.normalised_error(got, g["y"]) <= TOL["gemm_f32_3xtf32"]
    got = run_gemm_f32(B, g["a"], g["b"], cfg={"fp32_mode": 0}, status=status)
    assert O.normalised_error(got, g["y"]) <= TOL["gemm_f32_tf32"]


@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("mode", [0, 1])
def test_gemm_f32_transposes_ragged(B, status, ta, tb, mode):
    a, b = O.gemm_inputs(196, 132, 260, seed=21)
    want = O.gemm(a, b)
    got = run_gemm_f32(B, a.T.copy() if ta else a, b.T.copy() if tb else b, ta, tb, cfg={"fp32_mode": mode},
                       status=status)
    assert O.normalised_error(got, want) <= (TOL["gemm_f32_3xtf32"] if mode else TOL["gemm_f32_tf32"])


@pytest.mark.parametrize("cfg", [
    {"fp32_mode": 1}, {"fp32_mode": 1, "tile_n": 64}, {"fp32_mode": 1, "tile_n": 128, "stages": 2},
    {"fp32_mode": 0}, {"fp32_mode": 0, "cluster": 2, "tile_n": 128}, {"fp32_mode": 0, "tile_n": 64, "split_k": 4},
    {"fp32_mode": 0, "tile_n": 256, "raster": 2}, {"fp32_mode": 0, "raster": 3, "group_m": 4, "ctas": 74},
])
def test_gemm_f32_1024_every_knob(B, status, cfg):
    """The README task: C[1024,1024] = A.B, uniform[-1,1) inputs from seed 0."""
    a, b = O.gemm_inputs(1024, 1024, 1024, seed=0)
    want = O.gemm(a, b)
    got = run_gemm_f32(B, a, b, cfg=cfg, status=status)
    err = O.normalised_error(got, want)
    assert err <= (TOL["gemm_f32_3xtf32"] if cfg["fp32_mode"] else TOL["gemm_f32_tf32"]), err


def test_gemm_f32_tiny_and_k_tail(B, status):
    for (m, n, k) in [(1, 4, 4), (4, 8, 36), (129, 260, 100), (300, 36, 4)]:
        a, b = O.gemm_inputs(m, n, k, seed=m + n + k)
        got = run_gemm_f32(B, a, b, cfg={"fp32_mode": 1}, status=status)
        assert O.normalised_error(got, O.gemm(a, b)) <= TOL["gemm_f32_3xtf32"], (m, n, k)


def test_batched_gemm_f32(B, status):
    rng = np.random.default_rng(5)
    a = rng.uniform(-1, 1, (3, 72, 40)).astype(np.float32)
    b = rng.uniform(-1, 1, (3, 40, 56)).astype(np.float32)
    c = torch.full((3, 72, 56), float("nan"), device="cuda")
    B.bgemm_f32(dev(a), dev(b), c, cfg={"fp32_mode": 1}, status=status)
    assert O.normalised_error(c.cpu().numpy(), O.batch_gemm(a, b)) <= TOL["gemm_f32_3xtf32"]


def test_shapes_tma_cannot_address_run_on_the_cuda_core_kernel(B, status):
    """Row pitches that are not multiples of 16 bytes (K = 6 floats, bf16 N = 28, int8 K = 50):
    served by the CUDA-core kernel, same results."""
    for (m, n, k, ta, tb) in [(8, 8, 6, False, False), (70, 33, 45, False, True), (19, 27, 13, True, False)]:
        a, b = O.gemm_inputs(m, n, k, seed=m * n)
        got = run_gemm_f32(B, a.T.copy() if ta else a, b.T.copy() if tb else b, ta, tb, status=status)
        assert O.normalised_error(got, O.gemm(a, b)) <= 1e-5, (m, n, k)      # plain fp32 arithmetic here
    items = [O.batch_gemm_item(i, 28, 28, 1024, seed=35) for i in range(3)]   # the reference's (32, 28, 1024, 28) shape
    a = np.stack([i[0] for i in items])
    b = np.stack([i[1] for i in items])
    c = torch.full((3, 28, 28), float("nan"), device="cuda", dtype=torch.bfloat16)
    B.bgemm_bf16(bf16_dev(a), bf16_dev(b), c, status=status)
    assert O.bf16_output_ok(c.float().cpu().numpy(), O.batch_gemm(a, b))
    a8, b8 = O.gemm_int8_inputs(37, 20, 50, seed=36)
    assert (run_gemm_s8(B, a8, b8, status=status) == O.gemm_int8(a8, b8)).all()
    assert (run_gemm_s8(B, a8, b8.T.copy(), tb=True, status=status) == O.gemm_int8(a8, b8)).all()


def test_bad_arguments_are_refused(B):
    c = torch.zeros(8, 8, device="cuda")
    with pytest.raises(B.FtbError) as err:
        B.gemm_f32(torch.zeros(8, 8, device="cuda"), torch.zeros(8, 8, device="cuda"), c, cfg={"tile_n": 48})
    assert err.value.code == -3
    with pytest.raises(B.FtbError) as err:
        B.gemm_f32(torch.zeros(8, 6, device="cuda"), torch.zeros(6, 8, device="cuda"), c, cfg={"tile_n": 48})
    assert err.value.code == -3
    with pytest.raises(TypeError):
        B.gemm_f32(torch.zeros(8, 8), torch.zeros(8, 8, device="cuda"), c)


# ---------------------------------------------------------------- batched GEMM bf16
def test_bgemm_bf16_golden(B, status):
    g = _load("bgemm_bf16")
    a, b = O.from_bf16_bits(g["a_bits"]), O.from_bf16_bits(g["b_bits"])
    c = torch.full(g["y"].shape, float("nan"), device="cuda", dtype=torch.bfloat16)
    B.bgemm_bf16(bf16_dev(a), bf16_dev(b), c, status=status)
    assert O.bf16_output_ok(c.float().cpu().numpy(), g["y"])
    c32 = torch.full(g["y"].shape, float("nan"), device="cuda")
    B.bgemm_bf16(bf16_dev(a), bf16_dev(b), c32, status=status)
    assert O.normalised_error(c32.cpu().numpy(), g["y"]) <= TOL["bgemm_bf16_out_f32"]


@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("cfg", [{"cluster": 1}, {"cluster": 2, "tile_n": 256}, {"cluster": 2, "tile_n": 128, "stages": 3},
                                 {"cluster": 1, "tile_n": 64, "raster": 3, "group_m": 2}, {"cluster": 2, "tile_n": 512},
                                 {"cluster": 2, "tile_n": 512, "stages": 2, "raster": 2}])
def test_bgemm_bf16_layouts_and_tails(B, status, ta, tb, cfg):
    items = [O.batch_gemm_item(i, 328, 264, 136, seed=31) for i in range(3)]
    a = np.stack([i[0] for i in items])
    b = np.stack([i[1] for i in items])
    want = O.batch_gemm(a, b)
    a_in = np.ascontiguousarray(np.swapaxes(a, 1, 2)) if ta else a
    b_in = np.ascontiguousarray(np.swapaxes(b, 1, 2)) if tb else b
    c = torch.full(want.shape, float("nan"), device="cuda")
    B.bgemm_bf16(bf16_dev(a_in), bf16_dev(b_in), c, ta, tb, cfg=cfg, status=status)
    assert O.normalised_error(c.cpu().numpy(), want) <= TOL["bgemm_bf16_out_f32"]


def test_bgemm_bf16_full_size_properties(B, status):
    """B=64, M=N=K=2048 (the batch-sharded headline shape): two items against the oracle, every
    item through the row-sum identity (A.B).1 = A.(B.1), and run-to-run bit equality."""
    batch, n = 64, 2048
    a = torch.empty(batch, n, n, device="cuda", dtype=torch.bfloat16)
    b = torch.empty(batch, n, n, device="cuda", dtype=torch.bfloat16)
    host = {}
    for i in range(batch):
        ai, bi = O.batch_gemm_item(i, n, n, n, seed=3)
        a[i] = bf16_dev(ai)
        b[i] = bf16_dev(bi)
        if i in (0, 63):
            host[i] = (ai, bi)
    c = torch.full((batch, n, n), float("nan"), device="cuda", dtype=torch.bfloat16)
    B.bgemm_bf16(a, b, c, status=status)
    torch.cuda.synchronize()
    for i, (ai, bi) in host.items():
        assert O.bf16_output_ok(c[i].float().cpu().numpy(), O.gemm(ai, bi, out_dtype=np.float64))
    row_sums = c.double().sum(dim=2)
    want = torch.bmm(a.double(), b.double().sum(dim=2, keepdim=True)).squeeze(2)
    # 2048 bf16 roundings of magnitude <= 2^-9 |c| each, summed: well inside 2^-7 of the absolute row mass
    mass = c.double().abs().sum(dim=2)
    assert bool(((row_sums - want).abs() <= 2.0 ** -7 * mass).all())
    c2 = torch.empty_like(c)
    B.bgemm_bf16(a, b, c2, status=status)
    assert torch.equal(c, c2)


def test_bgemm_bf16_several_destinations(B, status):
    """One launch, the result in three buffers (stands for: the same slice of every rank's gathered
    output; here all three are local), each at its own batch offset of a larger buffer."""
    items = [O.batch_gemm_item(i, 200, 136, 72, seed=33) for i in range(2)]
    a = np.stack([i[0] for i in items])
    b = np.stack([i[1] for i in items])
    want = O.batch_gemm(a, b)
    full = [torch.full((5, 200, 136), float("nan"), device="cuda", dtype=torch.bfloat16) for _ in range(3)]
    offsets = [0, 1, 3]
    ptrs = [f[o:].data_ptr() for f, o in zip(full, offsets)]
    B.bgemm_bf16_multi(bf16_dev(a), bf16_dev(b), ptrs, 200, 136, cfg={"cluster": 2, "tile_n": 128}, status=status)
    torch.cuda.synchronize()
    for f, o in zip(full, offsets):
        assert O.bf16_output_ok(f[o:o + 2].float().cpu().numpy(), want)
        untouched = torch.cat([f[:o], f[o + 2:]])
        assert bool(torch.isnan(untouched.float()).all())            # nothing written outside the slice
    assert torch.equal(full[0][0:2], full[1][1:3]) and torch.equal(full[0][0:2], full[2][3:5])


def test_bgemm_bf16_eight_destinations_with_the_fused_gather_knobs(B, status):
    """What a rank of an 8-GPU job launches: its slice of the batch written to eight buffers at once (the
    maximum), with the knob set the multi-GPU path uses."""
    items = [O.batch_gemm_item(i, 512, 512, 256, seed=34) for i in range(3)]
    a = np.stack([i[0] for i in items])
    b = np.stack([i[1] for i in items])
    want = O.batch_gemm(a, b)
    full = [torch.full((4, 512, 512), float("nan"), device="cuda", dtype=torch.bfloat16) for _ in range(8)]
    ptrs = [f[d % 2:].data_ptr() for d, f in enumerate(full)]
    cfg = {"cluster": 2, "tile_n": 256, "raster": 3, "group_m": 4, "stages": 6, "release": 2}
    B.bgemm_bf16_multi(bf16_dev(a), bf16_dev(b), ptrs, 512, 512, cfg=cfg, status=status)
    torch.cuda.synchronize()
    for d, f in enumerate(full):
        got = f[d % 2:d % 2 + 3]
        assert O.bf16_output_ok(got.float().cpu().numpy(), want)
        assert torch.equal(got, full[0][0:3])
        rest = f[3:] if d % 2 == 0 else f[:1]
        assert bool(torch.isnan(rest.float()).all())
    with pytest.raises(ValueError):
        B.bgemm_bf16_multi(bf16_dev(a), bf16_dev(b), ptrs + ptrs[:1], 512, 512, cfg=cfg, status=status)


@pytest.mark.parametrize("shape", [(2, 512, 1024, 256), (3, 300, 1000, 200), (1, 1000, 776, 96), (2, 256, 520, 128)])
def test_bgemm_bf16_wide_pair_tile(B, status, shape):
    """The 256 x 512 pair tile (two accumulator halves per tile) gives the bits of the 256 x 256 tile,
    on whole tiles and on ragged M, N and K; the same through the several-destinations entry point
    and with fp32 output."""
    batch, m, n, k = shape
    items = [O.batch_gemm_item(i, m, n, k, seed=35) for i in range(batch)]
    a = bf16_dev(np.stack([i[0] for i in items]))
    b = bf16_dev(np.stack([i[1] for i in items]))
    want = O.batch_gemm(np.stack([i[0] for i in items]), np.stack([i[1] for i in items]))
    c256 = torch.full((batch, m, n), float("nan"), device="cuda", dtype=torch.bfloat16)
    c512 = torch.full_like(c256, float("nan"))
    B.bgemm_bf16(a, b, c256, cfg={"cluster": 2, "tile_n": 256}, status=status)
    B.bgemm_bf16(a, b, c512, cfg={"cluster": 2, "tile_n": 512}, status=status)
    torch.cuda.synchronize()
    assert torch.equal(c256, c512)
    assert O.bf16_output_ok(c512.float().cpu().numpy(), want)
    two = [torch.full_like(c256, float("nan")) for _ in range(2)]
    B.bgemm_bf16_multi(a, b, [t.data_ptr() for t in two], m, n, cfg={"cluster": 2, "tile_n": 512}, status=status)
    torch.cuda.synchronize()
    assert torch.equal(two[0], c512) and torch.equal(two[1], c512)
    c32 = torch.full((batch, m, n), float("nan"), device="cuda")
    B.bgemm_bf16(a, b, c32, cfg={"cluster": 2, "tile_n": 512}, status=status)
    assert O.normalised_error(c32.cpu().numpy(), want) <= TOL["bgemm_bf16_out_f32"]
    with pytest.raises(B.FtbError):                 # the wide tile exists for CTA pairs only
        B.bgemm_bf16(a, b, c512, cfg={"cluster": 1, "tile_n": 512}, status=status)
    assert int(status.item()) == 0


def test_gemm_f32_wide_pair_tile(B, status):
    a, b = O.gemm_inputs(520, 1100, 300, seed=36)
    want = O.gemm(a, b)
    for split_k in (1, 2):                          # split-K adds the halves' partial sums with atomics
        got = run_gemm_f32(B, a, b, cfg={"cluster": 2, "tile_n": 512, "fp32_mode": 0, "split_k": split_k}, status=status)
        assert O.normalised_error(got, want) <= TOL["gemm_f32_tf32"]
    with pytest.raises(B.FtbError):                 # no 3xTF32 on pairs, wide or not
        run_gemm_f32(B, a, b, cfg={"cluster": 2, "tile_n": 512, "fp32_mode": 1}, status=status)


@pytest.mark.parametrize("tile_n,cluster", [(512, 2), (256, 2), (128, 2), (256, 1), (64, 1)])
@pytest.mark.parametrize("stages", [2, 3, 4, 6])
@pytest.mark.parametrize("release", [1, 2])
def test_bgemm_bf16_pipeline_knobs_give_the_same_bits(B, status, tile_n, cluster, stages, release):
    """Every combination of tile, pipeline depth and stage hand-back (one by one, or two at a time)
    computes the same bf16 result as the library defaults, on a K long enough for several tiles'
    worth of ring wrap-arounds (K = 1184: 19 K blocks, an odd count)."""
    items = [O.batch_gemm_item(i, 520, 1040, 1184, seed=37) for i in range(3)]
    a = bf16_dev(np.stack([i[0] for i in items]))
    b = bf16_dev(np.stack([i[1] for i in items]))
    ref = torch.full((3, 520, 1040), float("nan"), device="cuda", dtype=torch.bfloat16)
    B.bgemm_bf16(a, b, ref, status=status)
    got = torch.full((3, 520, 1040), float("nan"), device="cuda", dtype=torch.bfloat16)
    cfg = {"tile_n": tile_n, "cluster": cluster, "stages": stages, "release": release}
    if B.validate(B.OP_BGEMM_BF16, cfg, 520, 1040, 1184) != 0:
        pytest.skip("this depth does not fit in shared memory with this tile")
    B.bgemm_bf16(a, b, got, cfg=cfg, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert torch.equal(got, ref)
    if (tile_n, stages, release) == (512, 4, 1):
        want = O.batch_gemm(np.stack([i[0] for i in items]), np.stack([i[1] for i in items]))
        assert O.bf16_output_ok(ref.float().cpu().numpy(), want)


def test_epilogues_agree(B, status):
    """The staged bulk-store epilogue and the per-thread store epilogue give the same bits."""
    items = [O.batch_gemm_item(i, 328, 264, 136, seed=34) for i in range(2)]
    a = bf16_dev(np.stack([i[0] for i in items]))
    b = bf16_dev(np.stack([i[1] for i in items]))
    c1 = torch.full((2, 328, 264), float("nan"), device="cuda", dtype=torch.bfloat16)
    c2 = torch.full((2, 328, 264), float("nan"), device="cuda", dtype=torch.bfloat16)
    B.bgemm_bf16(a, b, c1, status=status)
    B.bgemm_bf16(a, b, c2, cfg={"epilogue": 1}, status=status)
    torch.cuda.synchronize()
    assert torch.equal(c1, c2)


# ---------------------------------------------------------------- int8 GEMM
def run_gemm_s8(B, a, b, ta=False, tb=False, cfg=None, status=None):
    m = a.shape[1] if ta else a.shape[0]
    n = b.shape[0] if tb else b.shape[1]
    c = torch.full((m, n), -7, device="cuda", dtype=torch.int32)
    B.gemm_s8(dev(a), dev(b), c, ta, tb, cfg=cfg, status=status)
    torch.cuda.synchronize()
    return c.cpu().numpy()


def test_gemm_s8_golden_and_layouts(B, status):
    g = _load("gemm_int8")
    assert (run_gemm_s8(B, g["a"], g["b"], status=status) == g["y"]).all()
    a, b = O.gemm_int8_inputs(272, 384, 400, seed=41)
    want = O.gemm_int8(a, b)
    for ta in (False, True):
        for tb in (False, True):
            got = run_gemm_s8(B, a.T.copy() if ta else a, b.T.copy() if tb else b, ta, tb, status=status)
            assert (got == want).all(), (ta, tb)
    for cfg in ({"cluster": 2, "tile_n": 256}, {"cluster": 1, "tile_n": 128, "stages": 3}, {"raster": 2}, {"raster": 1},
                {"cluster": 2, "tile_n": 512}):
        assert (run_gemm_s8(B, a, b, cfg=cfg, status=status) == want).all(), cfg
    for tb in (False, True):                       # 256 x 512 tile, several tiles in both directions, ragged edges
        a2, b2 = O.gemm_int8_inputs(600, 1300, 272, seed=42)
        got = run_gemm_s8(B, a2, b2.T.copy() if tb else b2, False, tb, cfg={"cluster": 2, "tile_n": 512}, status=status)
        assert (got == O.gemm_int8(a2, b2)).all(), tb


def test_gemm_s8_extremes(B, status):
    k = 4096
    a = np.full((128, k), 127, dtype=np.int8)
    b = np.full((k, 256), -127, dtype=np.int8)
    assert (run_gemm_s8(B, a, b, status=status) == -127 * 127 * k).all()


def test_gemm_s8_8192_bit_exact(B, status):
    """M=N=K=8192, values uniform in [-127,127] from seed 4: a random 256x256 block against a
    literal int32 matmul, every row through the exact checksum C.1 = A.(B.1)."""
    n = 8192
    a, b = O.gemm_int8_inputs(n, n, n, seed=4)
    ad, bd = dev(a), dev(b)
    c = torch.full((n, n), -7, device="cuda", dtype=torch.int32)
    B.gemm_s8(ad, bd, c, status=status)
    torch.cuda.synchronize()
    r0, c0 = 3072 + 17, 5120 + 33
    block = c[r0:r0 + 256, c0:c0 + 256].cpu().numpy()
    assert (block == O.gemm_int8_direct(a[r0:r0 + 256], b[:, c0:c0 + 256])).all()
    b_row_sums = b.astype(np.int64).sum(axis=1)
    want = a.astype(np.int64) @ b_row_sums
    got = c.to(torch.int64).sum(dim=1).cpu().numpy()
    assert (got == want).all()
    c2 = torch.empty_like(c)
    B.gemm_s8(ad, bd, c2, cfg={"cluster": 1, "tile_n": 256}, status=status)
    assert torch.equal(c, c2)                      # another tiling, the same integers


# ---------------------------------------------------------------- conv2d
def run_conv(B, x, w, bias=None, stride=1, padding=0, dilation=1, groups=1, cfg=None, status=None):
    n, c, h, wd = x.shape
    k, _, r, s = w.shape
    p = O.out_size(h, r, stride, padding, dilation)
    q = O.out_size(wd, s, stride, padding, dilation)
    out = torch.full((n, k, p, q), float("nan"), device="cuda")
    ws = torch.empty(B.conv2d_workspace_bytes(n, c, h, wd, k, r, s, groups), dtype=torch.uint8, device="cuda")
    B.conv2d_nchw_f32(dev(x), dev(w), out, dev(bias) if bias is not None else None, (stride, stride),
                      (padding, padding), (dilation, dilation), groups, cfg=cfg, workspace=ws, status=status)
    torch.cuda.synchronize()
    return out.cpu().numpy()


def test_conv2d_golden(B, status):
    # the reference's own conv2d test case (flextensor/test/test_ops.py:85-115): 6 channels in 3 groups
    # (2 per group), 9 filters, stride 2, padding 1, dilation 2, bias
    g = _load("conv2d_grouped")
    stride, pad, dil, groups = (int(v) for v in g["params"])
    for mode, tol in ((0, TOL["conv2d_tf32"]), (1, TOL["conv2d_3xtf32"])):
        for extra in ({}, {"epilogue": 1}, {"split_k": 3}):
            cfg = dict(extra, fp32_mode=mode)
            got = run_conv(B, g["x"], g["w"], g["b"], stride, pad, dil, groups, cfg=cfg, status=status)
            assert got.shape == g["y"].shape
            assert O.normalised_error(got, g["y"]) <= tol, cfg
    assert int(status.item()) == 0
    g = _load("conv2d_3x3")
    for mode, tol in ((0, TOL["conv2d_tf32"]), (1, TOL["conv2d_3xtf32"])):
        got = run_conv(B, g["x"], g["w"], None, 1, 1, 1, 1, cfg={"fp32_mode": mode}, status=status)
        assert O.normalised_error(got, g["y"]) <= tol


@pytest.mark.parametrize("case", [
    dict(n=2, c=24, h=14, w=14, k=36, r=3, stride=1, pad=1, dil=1, groups=3, bias=True),
    dict(n=2, c=32, h=29, w=31, k=64, r=3, stride=2, pad=2, dil=2, groups=1, bias=True),
    dict(n=1, c=40, h=20, w=24, k=48, r=3, stride=1, pad=1, dil=1, groups=1, bias=False),
    dict(n=3, c=64, h=9, w=9, k=40, r=1, stride=1, pad=0, dil=1, groups=1, bias=False),
    dict(n=1, c=8, h=33, w=130, k=16, r=5, stride=1, pad=2, dil=1, groups=1, bias=True),
    dict(n=1, c=3, h=32, w=32, k=8, r=7, stride=2, pad=3, dil=1, groups=1, bias=False),
])
@pytest.mark.parametrize("mode", [0, 1])
def test_conv2d_cases(B, status, case, mode):
    x, w = O.conv2d_inputs(case["n"], case["c"], case["h"], case["w"], case["k"], case["r"], case["r"],
                           groups=case["groups"], seed=51)
    bias = np.random.default_rng(52).standard_normal(case["k"]).astype(np.float32) if case["bias"] else None
    want = O.conv2d_nchw(x, w, bias, case["stride"], case["pad"], case["dil"], case["groups"])
    got = run_conv(B, x, w, bias, case["stride"], case["pad"], case["dil"], case["groups"],
                   cfg={"fp32_mode": mode}, status=status)
    assert got.shape == want.shape
    assert O.normalised_error(got, want) <= (TOL["conv2d_3xtf32"] if mode else TOL["conv2d_tf32"])


@pytest.mark.parametrize("cfg", [{"fp32_mode": 0}, {"fp32_mode": 1}, {"fp32_mode": 0, "tile_n": 32},
                                 {"fp32_mode": 0, "tile_h": 1}, {"fp32_mode": 0, "split_k": 3},
                                 {"fp32_mode": 1, "split_k": 9, "tile_n": 32}])
def test_conv2d_resnet_stage2(B, status, cfg):
    """N=1, C=64, 56x56, K=64, 3x3, stride 1, pad 1; normal(0,1) input and weights from seed 1."""
    x, w = O.conv2d_inputs(1, 64, 56, 56, 64, 3, 3, seed=1)
    want = O.conv2d_nchw(x, w, None, 1, 1, 1, 1)
    got = run_conv(B, x, w, None, 1, 1, 1, 1, cfg=cfg, status=status)
    assert O.normalised_error(got, want) <= (TOL["conv2d_3xtf32"] if cfg["fp32_mode"] else TOL["conv2d_tf32"])


@pytest.mark.parametrize("shape", [(3, 64, 9, 9, 40, 1, 0), (1, 64, 56, 56, 64, 3, 1), (5, 16, 12, 10, 24, 3, 1)])
@pytest.mark.parametrize("cfg", [{"cluster": 2}, {"cluster": 2, "tile_n": 32, "split_k": 1}, {"cluster": 2, "split_k": 3},
                                 {"cluster": 1, "split_k": 1}])
def test_conv2d_cta_pairs(B, status, shape, cfg):
    """Two CTAs on two consecutive 128-pixel tiles (odd tile counts included)."""
    n, c, hw1, hw2, k, r, pad = shape
    x, w = O.conv2d_inputs(n, c, hw1, hw2, k, r, r, seed=53)
    want = O.conv2d_nchw(x, w, None, 1, pad, 1, 1)
    if cfg.get("split_k", 1) > r * r * ((c + 31) // 32):
        pytest.skip("more splits than K blocks")
    got = run_conv(B, x, w, None, 1, pad, 1, 1, cfg=dict(cfg, fp32_mode=0), status=status)
    assert O.normalised_error(got, want) <= TOL["conv2d_tf32"]


@pytest.mark.parametrize("shape", [
    # n, c, h, w, k, r, pad, dil
    (1, 64, 56, 56, 64, 3, 1, 1),      # bulk-store epilogue, filter taps split over CTAs
    (5, 64, 56, 56, 64, 3, 1, 1),      # more tiles than CTAs: slab ring and both accumulators wrap
    (2, 16, 128, 128, 40, 3, 1, 1),    # two tiles across the width, 40 of 48 accumulator columns used
    (2, 32, 14, 14, 48, 3, 1, 1),      # rows that bulk stores cannot address -> per-thread stores
    (1, 64, 56, 56, 64, 3, 2, 2),      # dilation 2
    (1, 8, 33, 130, 16, 5, 2, 1),      # 5x5, 25 taps
    (3, 40, 30, 30, 80, 3, 0, 1),      # no padding, channel count that is no multiple of 32
])
@pytest.mark.parametrize("cfg", [{"algo": 2}, {"algo": 2, "split_k": 3}, {"algo": 2, "tile_h": 1}, {"algo": 1}])
def test_conv2d_slab_algorithm(B, status, shape, cfg):
    """One input slab per channel chunk shared by all filter taps (algo 2) against the oracle and
    against the per-tap lowering (algo 1)."""
    n, c, h, wd, k, r, pad, dil = shape
    x, w = O.conv2d_inputs(n, c, h, wd, k, r, r, seed=57)
    bias = np.random.default_rng(58).standard_normal(k).astype(np.float32)
    want = O.conv2d_nchw(x, w, bias, 1, pad, dil, 1)
    got = run_conv(B, x, w, bias, 1, pad, dil, 1, cfg=dict(cfg, fp32_mode=0), status=status)
    assert got.shape == want.shape
    assert O.normalised_error(got, want) <= TOL["conv2d_tf32"]
    assert int(status.item()) == 0


@pytest.mark.parametrize("shape", [
    # n, c, h, w, k, r, pad, dil
    (5, 64, 56, 56, 64, 3, 1, 1),      # 64 accumulator columns, both accumulator pairs wrap
    (2, 96, 28, 28, 128, 3, 1, 1),     # 128 columns: the four accumulators fill tensor memory
    (1, 32, 40, 40, 48, 5, 2, 1),      # 25 taps
    (2, 64, 28, 28, 256, 3, 1, 1),     # 256 columns: one issuing thread only
])
@pytest.mark.parametrize("cfg", [{"algo": 2}, {"algo": 2, "split_k": 5}, {"algo": 2, "split_k": 9}, {"algo": 2, "split_k": 2},
                                 {"algo": 5}, {"algo": 2, "cluster": 2}, {"algo": 2, "gather": 2}, {"algo": 5, "gather": 2}])
def test_conv2d_slab_kernel_with_two_issuing_threads(B, status, shape, cfg):
    """Accumulators of at most 128 columns are filled by two MMA-issuing threads that take the taps of a slab
    alternately and are summed in the epilogue.  Tap shares of 2, 2, 2, 2, 1 (split 5: the last CTA has one
    thread's worth), of one tap each (split 9: single thread everywhere) and of 5 and 4 (split 2)."""
    n, c, h, wd, k, r, pad, dil = shape
    x, w = O.conv2d_inputs(n, c, h, wd, k, r, r, seed=61)
    bias = np.random.default_rng(62).standard_normal(k).astype(np.float32)
    want = O.conv2d_nchw(x, w, bias, 1, pad, dil, 1)
    try:
        got = run_conv(B, x, w, bias, 1, pad, dil, 1, cfg=dict(cfg, fp32_mode=0), status=status)
    except B.FtbError as exc:
        assert exc.code in (-2, -3), exc  # a knob set the shape cannot take is refused, never run wrong
        pytest.skip("refused: %s" % exc)
    assert got.shape == want.shape
    assert not np.isnan(got).any()
    assert O.normalised_error(got, want) <= TOL["conv2d_tf32"]
    assert int(status.item()) == 0


@pytest.mark.parametrize("shape", [
    # n, c, h, w, k, r, pad, dil
    (3, 128, 28, 28, 128, 3, 1, 1),    # 36 filter tiles of 16 KB: cannot stay resident
    (2, 256, 14, 14, 256, 3, 1, 1),    # 72 tiles of 32 KB
    (5, 64, 56, 56, 64, 3, 1, 1),      # would fit resident: streamed because asked for; ring and slabs wrap
    (2, 40, 20, 24, 200, 3, 1, 2),     # channel counts that are no multiples of 32, dilation 2
    (1, 96, 17, 19, 144, 5, 2, 1),     # 25 taps: stages of 5 taps (a filter row), rows bulk stores cannot address
    (2, 32, 30, 30, 72, 2, 0, 1),      # 2x2 filter, no padding
])
@pytest.mark.parametrize("cfg", [{"algo": 5}, {"algo": 5, "cluster": 1}, {"algo": 5, "cluster": 2}, {"algo": 5, "tile_h": 1},
                                 {"algo": 5, "epilogue": 1}, {"algo": 5, "relu": 1}])
def test_conv2d_slab_kernel_with_streamed_filter(B, status, shape, cfg):
    """The slab kernel with its filter passed through a ring of shared-memory stages (algo 5) instead of
    resident: against the oracle, on single CTAs and CTA pairs."""
    n, c, h, wd, k, r, pad, dil = shape
    x, w = O.conv2d_inputs(n, c, h, wd, k, r, r, seed=59)
    bias = np.random.default_rng(60).standard_normal(k).astype(np.float32)
    want = O.conv2d_nchw(x, w, bias, 1, pad, dil, 1)
    if cfg.get("relu"):
        want = np.maximum(want, 0)
    try:
        got = run_conv(B, x, w, bias, 1, pad, dil, 1, cfg=dict(cfg, fp32_mode=0), status=status)
    except B.FtbError as exc:
        assert exc.code in (-2, -3), exc
        pytest.skip("refused: %s" % exc)
    assert got.shape == want.shape
    assert not np.isnan(got).any()
    assert O.normalised_error(got, want) <= TOL["conv2d_tf32"], (shape, cfg)
    assert int(status.item()) == 0


@pytest.mark.parametrize("shape", [(2, 64, 8, 8, 48), (3, 32, 14, 14, 256), (1, 256, 56, 56, 64), (2, 20, 6, 6, 130)])
@pytest.mark.parametrize("cfg", [{}, {"algo": 3, "cluster": 1, "tile_n": 64, "split_k": 1}, {"algo": 3, "split_k": 2}, {"algo": 1},
                                 {"fp32_mode": 1}])
def test_conv2d_1x1_as_batched_gemm(B, status, shape, cfg):
    """A 1x1 filter (stride 1, no padding) is out[b] = W * in[b] on the NCHW tensors as they are."""
    n, c, h, wd, k = shape
    x, w = O.conv2d_inputs(n, c, h, wd, k, 1, 1, seed=61)
    bias = np.random.default_rng(62).standard_normal(k).astype(np.float32)
    want = O.conv2d_nchw(x, w, bias, 1, 0, 1, 1)
    if cfg.get("split_k", 1) > (c + 31) // 32:
        pytest.skip("more splits than K blocks")
    launches = B.launch_count()
    got = run_conv(B, x, w, bias, 1, 0, 1, 1, cfg=cfg, status=status)
    if cfg.get("algo", 0) != 1:                            # no layout pass in front of the kernel:
        used = B.launch_count() - launches                 # the GEMM alone, or a zeroing kernel and the GEMM
        assert used == 1 if cfg.get("split_k") == 1 else used <= 2
    assert O.normalised_error(got, want) <= (TOL["conv2d_3xtf32"] if cfg.get("fp32_mode") else TOL["conv2d_tf32"])
    with pytest.raises(B.FtbError):                        # padded or strided 1x1: not a plain GEMM
        run_conv(B, x, w, bias, 1, 1, 1, 1, cfg={"algo": 3}, status=status)


@pytest.mark.parametrize("shape", [
    # n, c, h, w, k, r, stride, pad, dil
    (1, 3, 64, 64, 64, 7, 2, 3, 1),      # RGB stem, 7x7 stride 2
    (2, 3, 30, 34, 24, 3, 1, 1, 1),      # 27 of 32 K entries real
    (1, 8, 19, 23, 40, 5, 1, 2, 2),      # 8 channels, dilation, 200 K entries -> 7 blocks
    (2, 1, 28, 28, 16, 5, 2, 0, 1),      # one channel, no padding
])
@pytest.mark.parametrize("cfg", [{}, {"algo": 4}, {"algo": 4, "split_k": 1, "tile_n": 32}, {"algo": 1}, {"algo": 4, "fp32_mode": 1}])
def test_conv2d_few_channels_as_im2col(B, status, shape, cfg):
    """Few input channels: a 1x1 conv over the im2col form (algo 4) against the oracle and the per-tap lowering."""
    n, c, h, wd, k, r, stride, pad, dil = shape
    x, w = O.conv2d_inputs(n, c, h, wd, k, r, r, seed=63)
    bias = np.random.default_rng(64).standard_normal(k).astype(np.float32)
    want = O.conv2d_nchw(x, w, bias, stride, pad, dil, 1)
    got = run_conv(B, x, w, bias, stride, pad, dil, 1, cfg=cfg, status=status)
    assert got.shape == want.shape
    assert O.normalised_error(got, want) <= (TOL["conv2d_3xtf32"] if cfg.get("fp32_mode") else TOL["conv2d_tf32"])
    assert int(status.item()) == 0
    x16, w16 = O.conv2d_inputs(1, 16, 12, 12, 8, 3, 3, seed=65)
    with pytest.raises(B.FtbError):                        # 16 channels: not this form
        run_conv(B, x16, w16, None, 1, 1, 1, 1, cfg={"algo": 4}, status=status)


@pytest.mark.parametrize("shape", [
    # n, c, h, w, k, stride, groups
    (2, 64, 14, 14, 96, 2, 1),      # even extent
    (3, 40, 15, 13, 48, 2, 1),      # odd extents: the last kept row and column are the image border
    (1, 32, 29, 31, 64, 3, 1),      # stride 3
    (2, 32, 12, 12, 32, 2, 2),      # two groups
])
@pytest.mark.parametrize("cfg", [{}, {"split_k": 1, "tile_n": 32}, {"fp32_mode": 1}])
def test_conv2d_strided_1x1_keeps_only_the_pixels_it_reads(B, status, shape, cfg):
    n, c, h, wd, k, stride, groups = shape
    x, w = O.conv2d_inputs(n, c, h, wd, k, 1, 1, groups=groups, seed=66)
    bias = np.random.default_rng(67).standard_normal(k).astype(np.float32)
    want = O.conv2d_nchw(x, w, bias, stride, 0, 1, groups)
    got = run_conv(B, x, w, bias, stride, 0, 1, groups, cfg=cfg, status=status)
    assert got.shape == want.shape
    assert O.normalised_error(got, want) <= (TOL["conv2d_3xtf32"] if cfg.get("fp32_mode") else TOL["conv2d_tf32"])
    assert int(status.item()) == 0


@pytest.mark.parametrize("shape", [
    # n, c, h, w, k, r, stride, pad, groups
    (16, 64, 7, 7, 96, 1, 1, 0, 1),      # two 49-pixel images per tile, 1x1
    (5, 32, 7, 7, 48, 3, 1, 1, 1),       # odd image count: the last tile holds one image
    (3, 16, 4, 4, 24, 3, 1, 1, 1),       # eight would fit, the batch has three
    (9, 32, 5, 3, 40, 1, 1, 0, 1),       # 15-pixel images, rows that bulk stores cannot address
    (6, 64, 14, 14, 32, 1, 2, 0, 1),     # strided 1x1 down to 7x7
    (4, 32, 6, 6, 32, 3, 1, 1, 2),       # two groups
])
@pytest.mark.parametrize("cfg", [{"algo": 1}, {"algo": 1, "split_k": 2}, {"algo": 1, "cluster": 2}, {"algo": 1, "fp32_mode": 1}])
def test_conv2d_small_images_share_a_tile(B, status, shape, cfg):
    """Images of at most 64 output pixels are packed several to a 128-row tile."""
    n, c, h, wd, k, r, stride, pad, groups = shape
    if cfg.get("split_k", 1) > r * r * ((c // groups + 31) // 32):
        pytest.skip("more splits than K blocks")
    x, w = O.conv2d_inputs(n, c, h, wd, k, r, r, groups=groups, seed=68)
    bias = np.random.default_rng(69).standard_normal(k).astype(np.float32)
    want = O.conv2d_nchw(x, w, bias, stride, pad, 1, groups)
    got = run_conv(B, x, w, bias, stride, pad, 1, groups, cfg=cfg, status=status)
    assert got.shape == want.shape
    assert O.normalised_error(got, want) <= (TOL["conv2d_3xtf32"] if cfg.get("fp32_mode") else TOL["conv2d_tf32"])
    assert int(status.item()) == 0


def _random_conv_cases(count, seed):
    import random
    rng = random.Random(seed)
    cases = []
    while len(cases) < count:
        groups = rng.choice([1, 1, 1, 2, 4])
        cg = rng.choice([1, 2, 3, 4, 5, 6, 8, 16, 32, 40]) if groups > 1 else rng.choice([1, 2, 3, 4, 5, 8, 12, 16, 24, 32, 40, 64])
        kg = rng.choice([1, 3, 8, 16, 24, 32, 48, 64, 100, 128])
        r = rng.choice([1, 1, 2, 3, 3, 3, 5, 7])
        s = r if rng.random() < 0.8 else rng.choice([1, 2, 3, 5])
        stride, dil, pad = rng.choice([1, 1, 1, 2, 2, 3]), rng.choice([1, 1, 1, 2]), rng.choice([0, 0, 1, 1, 2, 3])
        h = rng.randint(max(1, dil * (r - 1) + 1 - 2 * pad), 24)
        w = rng.randint(max(1, dil * (s - 1) + 1 - 2 * pad), 40)
        if rng.random() < 0.2:
            h = w = rng.choice([4, 7, 8, 14])
        n = rng.choice([1, 1, 2, 3, 5, 9])
        if O.out_size(h, r, stride, pad, dil) <= 0 or O.out_size(w, s, stride, pad, dil) <= 0:
            continue
        cfg = rng.choice([None, None, {"fp32_mode": 1}, {"algo": 1}, {"split_k": 1}])
        cases.append((n, cg * groups, h, w, kg * groups, r, s, stride, pad, dil, groups, rng.random() < 0.5, cfg))
    return cases


@pytest.mark.parametrize("case", _random_conv_cases(48, 7))
def test_conv2d_random_shapes_against_the_oracle(B, status, case):
    """Seeded random shapes through whatever algorithm the library picks for them (per-tap, slab, batched
    GEMM, im2col form, kept-pixel copy, several images per tile), each against the numpy oracle."""
    n, c, h, wd, k, r, s, stride, pad, dil, groups, with_bias, cfg = case
    x, w = O.conv2d_inputs(n, c, h, wd, k, r, s, groups=groups, seed=70)
    bias = np.random.default_rng(71).standard_normal(k).astype(np.float32) if with_bias else None
    want = O.conv2d_nchw(x, w, bias, stride, pad, dil, groups)
    got = run_conv(B, x, w, bias, stride, pad, dil, groups, cfg=cfg, status=status)
    assert got.shape == want.shape
    tol = TOL["conv2d_3xtf32"] if (cfg or {}).get("fp32_mode") else TOL["conv2d_tf32"]
    assert O.normalised_error(got, want) <= tol, case
    assert int(status.item()) == 0


# the reference's grouped benchmark shapes (flextensor/configs/grouped_config.py:1-6) plus small
# channel counts per group that are no multiple of 4
@pytest.mark.parametrize("shape", [(1, 1024, 14, 14, 512, 1, 1, 0, 4), (1, 1024, 14, 14, 512, 1, 1, 0, 8),
                                   (1, 1024, 14, 14, 512, 1, 1, 0, 16), (1, 1024, 14, 14, 512, 1, 1, 0, 32),
                                   (2, 30, 13, 12, 45, 3, 1, 1, 15), (3, 21, 9, 16, 14, 3, 2, 1, 7),
                                   (1, 10, 20, 20, 10, 3, 1, 1, 10), (2, 66, 8, 8, 33, 1, 1, 0, 11)])
def test_conv2d_groups_run_as_one_launch(B, status, shape):
    """Any number of channels per group, every group in the same launch: the layout pass plus one
    tensor-core kernel, whatever the group count."""
    n, c, h, wd, k, r, stride, pad, groups = shape
    x, w = O.conv2d_inputs(n, c, h, wd, k, r, r, groups=groups, seed=77)
    bias = np.random.default_rng(78).standard_normal(k).astype(np.float32)
    want = O.conv2d_nchw(x, w, bias, stride, pad, 1, groups)
    for cfg, tol in (({"fp32_mode": 0}, TOL["conv2d_tf32"]), ({"fp32_mode": 1}, TOL["conv2d_3xtf32"])):
        before = B.launch_count()
        got = run_conv(B, x, w, bias, stride, pad, 1, groups, cfg=cfg, status=status)
        assert B.launch_count() - before == 2, "layout pass + one conv kernel"
        assert O.normalised_error(got, want) <= tol, (shape, cfg)
    assert int(status.item()) == 0


@pytest.mark.parametrize("shape", [(5, 32, 20, 24, 48, 3, 1), (3, 64, 56, 56, 64, 3, 1), (1, 40, 9, 11, 20, 3, 1),
                                   (7, 16, 30, 130, 100, 5, 2), (2, 96, 14, 14, 256, 3, 1)])
@pytest.mark.parametrize("extra", [{}, {"split_k": 3}, {"epilogue": 1}])
def test_conv2d_slab_kernel_as_cta_pairs(B, status, shape, extra):
    """The slab kernel with two CTAs of a cluster on two consecutive tiles (cluster = 2): odd tile
    counts, split taps, both epilogues, against the oracle and against the single-CTA form."""
    n, c, h, wd, k, r, pad = shape
    x, w = O.conv2d_inputs(n, c, h, wd, k, r, r, seed=92)
    bias = np.random.default_rng(93).standard_normal(k).astype(np.float32)
    want = O.conv2d_nchw(x, w, bias, 1, pad, 1, 1)
    cfg = dict(extra, algo=2, cluster=2)
    try:
        got = run_conv(B, x, w, bias, 1, pad, 1, 1, cfg=cfg, status=status)
    except B.FtbError as exc:
        assert exc.code == -2 and extra.get("split_k")   # a split the resident filter cannot be cut into
        pytest.skip("this split does not fit the slab kernel")
    assert O.normalised_error(got, want) <= TOL["conv2d_tf32"]
    # with the taps split the same way both forms issue the same MMAs per output in the same order
    if "split_k" not in extra:
        try:
            single = run_conv(B, x, w, bias, 1, pad, 1, 1, cfg=dict(extra, algo=2, cluster=1, split_k=1), status=status)
            paired = run_conv(B, x, w, bias, 1, pad, 1, 1, cfg=dict(extra, algo=2, cluster=2, split_k=1), status=status)
        except B.FtbError as exc:
            assert exc.code == -2                    # the whole filter does not fit in one CTA's shared memory
        else:
            assert np.array_equal(paired, single)
    assert int(status.item()) == 0


@pytest.mark.parametrize("shape", [
    # n, c, h, w, k, r, pad, dil
    (5, 64, 56, 56, 64, 3, 1, 1),      # resident filter, slab ring and both accumulators wrap
    (3, 128, 28, 28, 128, 3, 1, 1),    # streamed filter
    (2, 40, 20, 24, 200, 3, 1, 2),     # channel counts that are no multiples of 32 (zero-filled chunk tail), dilation 2
    (1, 8, 33, 130, 16, 5, 2, 1),      # 5x5, two tiles across the width, few channels
    (2, 32, 14, 14, 48, 3, 1, 1),      # small planes, per-thread epilogue
    (3, 20, 9, 7, 24, 3, 0, 1),        # no padding, a slab narrower than a warp's 32 pixels
])
@pytest.mark.parametrize("cfg", [{"algo": 2, "gather": 2}, {"algo": 2, "gather": 2, "cluster": 2}, {"algo": 5, "gather": 2},
                                 {"algo": 2, "gather": 2, "split_k": 3}, {"algo": 2, "gather": 2, "relu": 1}])
def test_conv2d_slab_kernel_gathers_its_slabs_from_nchw(B, status, shape, cfg):
    """gather = 2: no channels-last copy; loader warps of the slab kernel build every slab from the NCHW
    tensor (zero-filling padding, channel tails and, in a pair with an odd tile count, the tile past the end)."""
    n, c, h, wd, k, r, pad, dil = shape
    x, w = O.conv2d_inputs(n, c, h, wd, k, r, r, seed=61)
    bias = np.random.default_rng(62).standard_normal(k).astype(np.float32)
    want = O.conv2d_nchw(x, w, bias, 1, pad, dil, 1)
    if cfg.get("relu"):
        want = np.maximum(want, 0)
    try:
        got = run_conv(B, x, w, bias, 1, pad, dil, 1, cfg=dict(cfg, fp32_mode=0), status=status)
    except B.FtbError as exc:
        assert exc.code in (-2, -3), exc
        pytest.skip("refused: %s" % exc)
    assert got.shape == want.shape
    assert not np.isnan(got).any()
    assert O.normalised_error(got, want) <= TOL["conv2d_tf32"], (shape, cfg)
    # the same MMAs on the same operand bits as the layout-pass form; only where the library splits the taps
    # over CTAs do partial sums meet in a different order
    plain = run_conv(B, x, w, bias, 1, pad, dil, 1, cfg=dict(cfg, fp32_mode=0, gather=1), status=status)
    assert O.normalised_error(got, plain) <= 1e-5
    assert int(status.item()) == 0


def test_conv2d_slab_algorithm_refuses_what_it_cannot_take(B, status):
    x, w = O.conv2d_inputs(1, 32, 16, 16, 32, 3, 3, seed=59)
    for kwargs, cfg in ((dict(stride=2), {"algo": 2}),                 # stride 2
                        (dict(stride=1), {"algo": 2, "fp32_mode": 1}),  # 3xTF32
                        (dict(stride=1), {"algo": 2, "tile_n": 16}),                # not a tile width
                        (dict(stride=1), {"algo": 3}),                             # GEMM form of a 3x3
                        (dict(stride=1), {"algo": 5, "split_k": 3}),               # a streamed filter is never split
                        (dict(stride=1), {"algo": 6})):
        with pytest.raises(B.FtbError):
            run_conv(B, x, w, None, kwargs["stride"], 1, 1, 1, cfg=cfg, status=status)
    xg, wg = O.conv2d_inputs(1, 32, 16, 16, 32, 3, 3, groups=2, seed=59)
    with pytest.raises(B.FtbError):
        run_conv(B, xg, wg, None, 1, 1, 1, 2, cfg={"algo": 2}, status=status)


def test_conv2d_workspace_is_required(B):
    x = torch.zeros(1, 8, 8, 8, device="cuda")
    w = torch.zeros(8, 8, 3, 3, device="cuda")
    out = torch.zeros(1, 8, 6, 6, device="cuda")
    with pytest.raises(ValueError):
        B.conv2d_nchw_f32(x, w, out, workspace=torch.empty(16, dtype=torch.uint8, device="cuda"))
    rc = B.lib().ftb_conv2d_nchw_f32(x.data_ptr(), w.data_ptr(), None, out.data_ptr(), 1, 8, 8, 8, 8, 3, 3, 1, 1, 0,
                                     0, 1, 1, 1, None, None, 0, None, None)
    assert rc == -4


# ---------------------------------------------------------------- depthwise conv2d
def run_dw(B, x, w, bias=None, stride=1, padding=0, dilation=1, cfg=None):
    n, c, h, wd = x.shape
    _, f, r, s = w.shape
    p = O.out_size(h, r, stride, padding, dilation)
    q = O.out_size(wd, s, stride, padding, dilation)
    out = torch.full((n, c * f, p, q), float("nan"), device="cuda")
    B.dwconv2d_nchw_f32(dev(x), dev(w), out, dev(bias) if bias is not None else None, (stride, stride),
                        (padding, padding), (dilation, dilation), cfg=cfg)
    torch.cuda.synchronize()
    return out.cpu().numpy()


def test_depthwise_golden(B):
    g = _load("depthwise_f3")
    stride, pad, dil = (int(v) for v in g["params"])
    got = run_dw(B, g["x"], g["w"], g["b"], stride, pad, dil)
    assert O.normalised_error(got, g["y"]) <= TOL["depthwise_f32"]


@pytest.mark.parametrize("cfg", [None, {"tile_h": 4}, {"tile_h": 8, "threads": 256}, {"tile_h": 7},
                                 {"tile_h": 14, "threads": 128}, {"tile_h": 56, "threads": 512},
                                 {"tile_h": 1, "threads": 64}])
def test_depthwise_c256_56(B, cfg):
    """N=1, C=256, 56x56, 3x3, stride 1, pad 1, multiplier 1; uniform[-1,1) from seed 2."""
    x, w = O.depthwise_inputs(1, 256, 56, 56, 1, 3, 3, seed=2)
    got = run_dw(B, x, w, None, 1, 1, 1, cfg=cfg)
    assert O.normalised_error(got, O.depthwise_conv2d_nchw(x, w, None, 1, 1, 1)) <= TOL["depthwise_f32"]


@pytest.mark.parametrize("shape", [(2, 6, 19, 23, 2, 5, 2, 3, 2), (1, 32, 112, 112, 1, 3, 1, 1, 1),
                                   (8, 16, 112, 112, 6, 3, 2, 1, 1), (2, 160, 7, 7, 6, 3, 1, 1, 1),
                                   (1, 3, 5, 5, 1, 3, 1, 0, 1), (1, 4, 30, 33, 1, 7, 1, 3, 1),
                                   (2, 8, 21, 24, 3, 3, 1, 1, 1), (1, 5, 9, 132, 1, 3, 1, 1, 1)])
def test_depthwise_shapes(B, shape):
    n, c, h, w_, f, r, stride, pad, dil = shape
    x, w = O.depthwise_inputs(n, c, h, w_, f, r, r, seed=61)
    bias = np.random.default_rng(62).standard_normal(c * f).astype(np.float32)
    got = run_dw(B, x, w, bias, stride, pad, dil)
    want = O.depthwise_conv2d_nchw(x, w, bias, stride, pad, dil)
    assert got.shape == want.shape
    assert O.normalised_error(got, want) <= TOL["depthwise_f32"]


@pytest.mark.parametrize("shape", [(2, 12, 17, 19, 2, 5, 1, 2), (3, 9, 28, 28, 1, 5, 2, 2), (1, 7, 13, 13, 1, 3, 2, 0),
                                   (4, 64, 14, 14, 1, 3, 2, 1), (2, 5, 6, 50, 3, 3, 1, 1)])
@pytest.mark.parametrize("cfg", [None, {"threads": 256}, {"tile_h": 4}])
def test_depthwise_window_kernel_and_staged_kernel_agree(B, shape, cfg):
    """3x3 / 5x5 at stride 1 or 2: the window kernel (default) and the staged kernel (a strip height is
    given) against the oracle."""
    n, c, h, w_, f, r, stride, pad = shape
    x, w = O.depthwise_inputs(n, c, h, w_, f, r, r, seed=63)
    bias = np.random.default_rng(64).standard_normal(c * f).astype(np.float32)
    got = run_dw(B, x, w, bias, stride, pad, 1, cfg=cfg)
    want = O.depthwise_conv2d_nchw(x, w, bias, stride, pad, 1)
    assert got.shape == want.shape
    assert O.normalised_error(got, want) <= TOL["depthwise_f32"]


def _random_depthwise_cases(count, seed):
    import random
    rng = random.Random(seed)
    cases = []
    while len(cases) < count:
        c, f = rng.choice([1, 3, 8, 17, 32, 64]), rng.choice([1, 1, 2, 3])
        r = rng.choice([1, 3, 3, 3, 5, 5, 7])
        stride, dil, pad = rng.choice([1, 1, 2, 3]), rng.choice([1, 1, 1, 2]), rng.choice([0, 1, 1, 2, 3])
        h = rng.randint(max(1, dil * (r - 1) + 1 - 2 * pad), 30)
        w = rng.choice([8, 16, 28, 56]) if rng.random() < 0.3 else rng.randint(max(1, dil * (r - 1) + 1 - 2 * pad), 50)
        if O.out_size(h, r, stride, pad, dil) <= 0 or O.out_size(w, r, stride, pad, dil) <= 0:
            continue
        cfg = rng.choice([None, None, None, {"tile_h": 4}, {"tile_h": 8}, {"threads": 256}, {"tile_h": 2, "threads": 64}])
        cases.append((rng.choice([1, 2, 5]), c, h, w, f, r, stride, pad, dil, cfg))
    return cases


@pytest.mark.parametrize("case", _random_depthwise_cases(36, 11))
def test_depthwise_random_shapes_against_the_oracle(B, case):
    n, c, h, w_, f, r, stride, pad, dil, cfg = case
    x, w = O.depthwise_inputs(n, c, h, w_, f, r, r, seed=72)
    bias = np.random.default_rng(73).standard_normal(c * f).astype(np.float32)
    got = run_dw(B, x, w, bias, stride, pad, dil, cfg=cfg)
    want = O.depthwise_conv2d_nchw(x, w, bias, stride, pad, dil)
    assert got.shape == want.shape
    assert O.normalised_error(got, want) <= TOL["depthwise_f32"], case


def _random_gemm_cases(count, seed):
    import random
    rng = random.Random(seed)
    cases = []
    for _ in range(count):
        cfg = rng.choice([None, None, None, {"cluster": 1, "tile_n": 64}, {"cluster": 2, "tile_n": 128},
                          {"cluster": 2, "tile_n": 512}, {"cluster": 1, "tile_n": 256, "stages": 2}])
        cases.append((rng.choice(["tf32", "3xtf32", "bf16", "s8"]), rng.choice([1, 7, 64, 100, 128, 200, 256, 384, 520]),
                      rng.choice([4, 8, 36, 64, 100, 128, 256, 520, 1000]), rng.choice([4, 8, 20, 32, 64, 100, 256, 520]),
                      rng.random() < 0.3, rng.random() < 0.3, cfg))
    return cases


@pytest.mark.parametrize("case", _random_gemm_cases(40, 13))
def test_gemm_random_shapes_against_the_oracle(B, status, case):
    """Seeded random shapes, majors and knobs over the three GEMM entry points, including operands that only
    the CUDA-core kernel can address; a knob set the library refuses must be refused with a config error."""
    kind, m, n, k, ta, tb, cfg = case
    try:
        if kind in ("tf32", "3xtf32"):
            a, b = O.gemm_inputs(m, n, k, seed=74)
            got = run_gemm_f32(B, a.T.copy() if ta else a, b.T.copy() if tb else b, ta, tb,
                               cfg=dict(cfg or {}, fp32_mode=1 if kind == "3xtf32" else 0), status=status)
            assert O.normalised_error(got, O.gemm(a, b)) <= TOL["gemm_f32_3xtf32" if kind == "3xtf32" else "gemm_f32_tf32"], case
        elif kind == "bf16":
            items = [O.batch_gemm_item(i, m, n, k, seed=75) for i in range(2)]
            a, b = np.stack([i[0] for i in items]), np.stack([i[1] for i in items])
            c = torch.full((2, m, n), float("nan"), device="cuda")
            B.bgemm_bf16(bf16_dev(np.ascontiguousarray(np.swapaxes(a, 1, 2)) if ta else a),
                         bf16_dev(np.ascontiguousarray(np.swapaxes(b, 1, 2)) if tb else b), c, ta, tb, cfg=cfg, status=status)
            assert O.normalised_error(c.cpu().numpy(), O.batch_gemm(a, b)) <= TOL["bgemm_bf16_out_f32"], case
        else:
            a, b = O.gemm_int8_inputs(m, n, k, seed=76)
            got = run_gemm_s8(B, a.T.copy() if ta else a, b.T.copy() if tb else b, ta, tb, cfg=cfg, status=status)
            assert (got == O.gemm_int8(a, b)).all(), case
    except B.FtbError as err:
        assert cfg is not None and err.code == -3, case
    assert int(status.item()) == 0


def test_a_wait_that_runs_out_is_reported_not_hung(B):
    """A barrier nothing completes: the bounded wait gives up, the status word says so, and the
    device keeps working afterwards."""
    st = B.new_status()
    B.selftest_bounded_wait(st)
    torch.cuda.synchronize()
    assert int(st.item()) == 1
    with pytest.raises(RuntimeError, match="gave up waiting"):
        B.check_status(st)
    a, b = O.gemm_inputs(64, 64, 64, seed=1)
    got = run_gemm_f32(B, a, b, cfg={"fp32_mode": 1})
    assert O.normalised_error(got, O.gemm(a, b)) <= TOL["gemm_f32_3xtf32"]


def test_launch_counter_counts_our_kernels(B):
    before = B.launch_count()
    x, w = O.depthwise_inputs(1, 4, 8, 8, 1, 3, 3)
    run_dw(B, x, w, None, 1, 1, 1)
    assert B.launch_count() == before + 1
