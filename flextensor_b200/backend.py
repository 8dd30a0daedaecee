"""ctypes binding of the C ABI in ``include/ftb200.h`` plus thin torch-tensor launchers.

This is the only place Python touches the native library.  There is no CPU or
library fallback: if the shared object is missing, or the current device is not
sm_100, the calls raise.
"""
import ctypes
import os
import threading

import torch

# FTB200_LIBRARY may name another build of the same library (e.g. the wait-profiling build that
# `python -m flextensor_b200.build --profile-waits` writes next to the product one).
_LIB_PATH = os.environ.get("FTB200_LIBRARY") or os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib",
                                                             "libftb200.so")
_lib = None
_lib_lock = threading.Lock()

OP_GEMM_F32, OP_BGEMM_BF16, OP_GEMM_S8, OP_CONV2D, OP_DWCONV2D = range(5)

# bits a kernel may set in the device status word (a bounded in-kernel wait ran out)
DEV_STATUS_BITS = {
    1: "MMA issuer gave up waiting for a TMA stage",
    2: "TMA producer gave up waiting for a free stage",
    4: "epilogue gave up waiting for an accumulator",
    8: "MMA issuer gave up waiting for a free accumulator",
    16: "wait on the 3xTF32 split stage ran out",
}


class FtbConfig(ctypes.Structure):
    """Mirror of ``struct ftb_config``; 0 in a field means "library default"."""

    _fields_ = [
        ("tile_n", ctypes.c_int32),
        ("stages", ctypes.c_int32),
        ("raster", ctypes.c_int32),
        ("group_m", ctypes.c_int32),
        ("split_k", ctypes.c_int32),
        ("fp32_mode", ctypes.c_int32),
        ("ctas", ctypes.c_int32),
        ("tile_h", ctypes.c_int32),
        ("threads", ctypes.c_int32),
        ("cluster", ctypes.c_int32),
        ("algo", ctypes.c_int32),
        ("epilogue", ctypes.c_int32),
        ("release", ctypes.c_int32),
        ("relu", ctypes.c_int32),
        ("gather", ctypes.c_int32),
        ("reserved", ctypes.c_int32 * 1),
    ]

    KNOBS = ("tile_n", "stages", "raster", "group_m", "split_k", "fp32_mode", "ctas", "tile_h", "threads",
             "cluster", "algo", "epilogue", "release", "relu", "gather")

    @classmethod
    def from_dict(cls, knobs):
        cfg = cls()
        for name, value in (knobs or {}).items():
            if name == "_diag":  # diagnostic builds of the library only
                cfg.reserved[0] = int(value)
                continue
            if name not in cls.KNOBS:
                raise KeyError("unknown kernel knob %r" % (name,))
            setattr(cfg, name, int(value))
        return cfg

    def to_dict(self):
        return {name: int(getattr(self, name)) for name in self.KNOBS}


class FtbError(RuntimeError):
    """A launcher returned a negative FTB_E_* code (``.code``)."""

    def __init__(self, code, where, message=None):
        self.code = code
        self.where = where
        if message is None:
            detail = lib().ftb_strerror(code).decode()
            cuda = lib().ftb_last_cuda_error()
            message = "%s failed: %s (code %d, last CUDA error %d)" % (where, detail, code, cuda)
        super().__init__(message)

    def __reduce__(self):  # crosses process boundaries (measurement workers)
        return (FtbError, (self.code, self.where, str(self)))


def lib_path():
    return _LIB_PATH


def lib():
    """Load (once) and return the native library; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    with _lib_lock:
        if _lib is not None:
            return _lib
        if not os.path.exists(_LIB_PATH):
            raise RuntimeError(
                "native library %s is missing: build it with `python -m flextensor_b200.build`; "
                "there is no fallback path" % _LIB_PATH)
        handle = ctypes.CDLL(_LIB_PATH)
        i64, i32, vp = ctypes.c_int64, ctypes.c_int, ctypes.c_void_p
        cfgp = ctypes.POINTER(FtbConfig)
        handle.ftb_version.restype = i32
        handle.ftb_version.argtypes = []
        handle.ftb_strerror.restype = ctypes.c_char_p
        handle.ftb_strerror.argtypes = [i32]
        handle.ftb_last_cuda_error.restype = i32
        handle.ftb_last_cuda_error.argtypes = []
        handle.ftb_device_check.restype = i32
        handle.ftb_device_check.argtypes = []
        handle.ftb_launch_count.restype = i64
        handle.ftb_launch_count.argtypes = []
        handle.ftb_validate.restype = i32
        handle.ftb_validate.argtypes = [i32, cfgp, i64, i64, i64]
        handle.ftb_debug_wait_profile.restype = i32
        handle.ftb_debug_wait_profile.argtypes = [ctypes.POINTER(ctypes.c_uint64), i32]
        handle.ftb_selftest_bounded_wait.restype = i32
        handle.ftb_selftest_bounded_wait.argtypes = [vp, vp]
        handle.ftb_gemm_f32.restype = i32
        handle.ftb_gemm_f32.argtypes = [vp, vp, vp, i64, i64, i64, i32, i32, cfgp, vp, vp]
        handle.ftb_bgemm_f32.restype = i32
        handle.ftb_bgemm_f32.argtypes = [vp, vp, vp, i64, i64, i64, i64, i32, i32, cfgp, vp, vp]
        handle.ftb_bgemm_bf16.restype = i32
        handle.ftb_bgemm_bf16.argtypes = [vp, vp, vp, i64, i64, i64, i64, i32, i32, i32, cfgp, vp, vp]
        handle.ftb_bgemm_bf16_multi.restype = i32
        handle.ftb_bgemm_bf16_multi.argtypes = [vp, vp, ctypes.POINTER(vp), i32, i64, i64, i64, i64, i32, i32, i32,
                                                cfgp, vp, vp]
        handle.ftb_gemm_s8.restype = i32
        handle.ftb_gemm_s8.argtypes = [vp, vp, vp, i64, i64, i64, i32, i32, cfgp, vp, vp]
        handle.ftb_conv2d_workspace_bytes.restype = ctypes.c_size_t
        handle.ftb_conv2d_workspace_bytes.argtypes = [i64] * 8
        handle.ftb_conv2d_nchw_f32.restype = i32
        handle.ftb_conv2d_nchw_f32.argtypes = ([vp] * 4 + [i64] * 7 + [i32] * 7 +
                                               [cfgp, vp, ctypes.c_size_t, vp, vp])
        handle.ftb_conv2d_pack_filter.restype = i32
        handle.ftb_conv2d_pack_filter.argtypes = [vp] + [i64] * 7 + [i32] * 7 + [cfgp, vp, ctypes.c_size_t, vp]
        handle.ftb_conv2d_nchw_f32_prepacked.restype = i32
        handle.ftb_conv2d_nchw_f32_prepacked.argtypes = ([vp] * 4 + [i64] * 7 + [i32] * 7 +
                                                         [cfgp, vp, ctypes.c_size_t, vp, vp])
        handle.ftb_conv2d_nchw_f32_multi.restype = i32
        handle.ftb_conv2d_nchw_f32_multi.argtypes = ([vp] * 3 + [ctypes.POINTER(vp), i32] + [i64] * 7 + [i32] * 8 +
                                                     [cfgp, vp, ctypes.c_size_t, vp, vp])
        handle.ftb_conv2d_nhwc_workspace_bytes.restype = ctypes.c_size_t
        handle.ftb_conv2d_nhwc_workspace_bytes.argtypes = [i64] * 5
        handle.ftb_conv2d_nhwc_f32.restype = i32
        handle.ftb_conv2d_nhwc_f32.argtypes = ([vp] * 4 + [i64] * 7 + [i32] * 8 + [cfgp, vp, ctypes.c_size_t, vp, vp])
        handle.ftb_conv3d_workspace_bytes.restype = ctypes.c_size_t
        handle.ftb_conv3d_workspace_bytes.argtypes = [i64] * 10
        handle.ftb_conv3d_ncdhw_f32.restype = i32
        handle.ftb_conv3d_ncdhw_f32.argtypes = ([vp] * 4 + [i64] * 9 + [ctypes.POINTER(i32)] * 3 + [i32, i32] +
                                                [cfgp, vp, ctypes.c_size_t, vp, vp])
        handle.ftb_conv2d_nchw_f32_noalloc.restype = i32
        handle.ftb_conv2d_nchw_f32_noalloc.argtypes = [vp] * 4 + [i64] * 7 + [i32] * 7 + [cfgp, vp, vp]
        handle.ftb_dwconv2d_nchw_f32.restype = i32
        handle.ftb_dwconv2d_nchw_f32.argtypes = [vp] * 4 + [i64] * 7 + [i32] * 6 + [cfgp, vp, vp]
        handle.ftb_dwconv2d_nchw_f32_multi.restype = i32
        handle.ftb_dwconv2d_nchw_f32_multi.argtypes = ([vp] * 3 + [ctypes.POINTER(vp), i32] + [i64] * 7 + [i32] * 6 +
                                                       [cfgp, vp, vp])
        _lib = handle
    return _lib


EXPORTED_SYMBOLS = (
    "ftb_version", "ftb_strerror", "ftb_last_cuda_error", "ftb_device_check", "ftb_validate",
    "ftb_launch_count", "ftb_selftest_bounded_wait", "ftb_debug_wait_profile", "ftb_gemm_f32", "ftb_bgemm_f32", "ftb_bgemm_bf16", "ftb_bgemm_bf16_multi", "ftb_gemm_s8",
    "ftb_conv2d_workspace_bytes", "ftb_conv2d_nchw_f32", "ftb_conv2d_nchw_f32_noalloc", "ftb_dwconv2d_nchw_f32",
    "ftb_dwconv2d_nchw_f32_multi", "ftb_conv2d_nchw_f32_multi", "ftb_conv2d_pack_filter",
    "ftb_conv2d_nchw_f32_prepacked", "ftb_conv3d_workspace_bytes", "ftb_conv3d_ncdhw_f32",
    "ftb_conv2d_nhwc_f32", "ftb_conv2d_nhwc_workspace_bytes",
)


def _cfg_ptr(cfg):
    if cfg is None:
        return None
    if isinstance(cfg, dict):
        cfg = FtbConfig.from_dict(cfg)
    return ctypes.byref(cfg)


def _check(t, dtype, name):
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise TypeError("%s must be a CUDA tensor" % name)
    if t.dtype != dtype:
        raise TypeError("%s must have dtype %s, got %s" % (name, dtype, t.dtype))
    if not t.is_contiguous():
        raise ValueError("%s must be contiguous" % name)


def _stream_ptr(stream):
    s = stream if stream is not None else torch.cuda.current_stream()
    return ctypes.c_void_p(s.cuda_stream)


def _status_ptr(status):
    if status is None:
        return None
    _check(status, torch.int32, "status")
    return ctypes.c_void_p(status.data_ptr())


def new_status(device=None):
    """A zeroed device int the kernels report bounded-wait failures into."""
    return torch.zeros(1, dtype=torch.int32, device=device or "cuda")


def check_status(status):
    """Synchronising read of a status word; raises if any kernel gave up a wait."""
    bits = int(status.item())
    if bits:
        why = [text for bit, text in DEV_STATUS_BITS.items() if bits & bit]
        raise RuntimeError("kernel reported status %d: %s" % (bits, "; ".join(why)))


def validate(op, cfg, m, n, k):
    if isinstance(cfg, dict):
        cfg = FtbConfig.from_dict(cfg)
    return int(lib().ftb_validate(op, ctypes.byref(cfg) if cfg is not None else None, m, n, k))


def launch_count():
    return int(lib().ftb_launch_count())


WAIT_PROFILE_SLOTS = ("producer_wait_empty", "issuer_wait_full", "issuer_wait_tmem_free", "epilogue_wait_tmem_full",
                      "producer_loop", "issuer_loop", "epilogue_loop", "ctas", "epilogue_tmem_ld",
                      "epilogue_bulk_wait", "epilogue_stage", "epilogue_store_issue", "epilogue_vote", "unused13",
                      "unused14", "unused15")


def wait_profile(reset=True):
    """Cycle counters of a wait-profiling build (``FTB200_LIBRARY`` pointing at it) as a dict;
    raises ``FtbError`` (unsupported) on the product build."""
    arr = (ctypes.c_uint64 * 16)()
    rc = lib().ftb_debug_wait_profile(arr, int(reset))
    if rc:
        raise FtbError(rc, "ftb_debug_wait_profile")
    return dict(zip(WAIT_PROFILE_SLOTS, (int(v) for v in arr)))


def selftest_bounded_wait(status, stream=None):
    """Launch the wait self-test (about two seconds on the device); ``status`` gets bit 1."""
    with torch.cuda.device(status.device):
        rc = lib().ftb_selftest_bounded_wait(_status_ptr(status), _stream_ptr(stream))
    if rc:
        raise FtbError(rc, "ftb_selftest_bounded_wait")


def gemm_f32(a, b, c, trans_a=False, trans_b=False, cfg=None, status=None, stream=None):
    """c[M,N] = op(a) @ op(b) in fp32 on TF32 tensor cores (3xTF32 when cfg.fp32_mode == 1)."""
    for t, nm in ((a, "a"), (b, "b"), (c, "c")):
        _check(t, torch.float32, nm)
    m, n = c.shape
    k = a.shape[0] if trans_a else a.shape[1]
    if tuple(a.shape) != ((k, m) if trans_a else (m, k)) or tuple(b.shape) != ((n, k) if trans_b else (k, n)):
        raise ValueError("gemm_f32: shapes do not agree: %s %s -> %s" % (a.shape, b.shape, c.shape))
    with torch.cuda.device(c.device):
        rc = lib().ftb_gemm_f32(a.data_ptr(), b.data_ptr(), c.data_ptr(), m, n, k, int(trans_a), int(trans_b),
                                _cfg_ptr(cfg), _status_ptr(status), _stream_ptr(stream))
    if rc:
        raise FtbError(rc, "ftb_gemm_f32")


def bgemm_f32(a, b, c, trans_a=False, trans_b=False, cfg=None, status=None, stream=None):
    """c[B,M,N] = op(a[b]) @ op(b[b]) in fp32 on TF32 tensor cores (3xTF32 when cfg.fp32_mode == 1)."""
    for t, nm in ((a, "a"), (b, "b"), (c, "c")):
        _check(t, torch.float32, nm)
    batch, m, n = c.shape
    k = a.shape[1] if trans_a else a.shape[2]
    if (tuple(a.shape) != ((batch, k, m) if trans_a else (batch, m, k)) or
            tuple(b.shape) != ((batch, n, k) if trans_b else (batch, k, n))):
        raise ValueError("bgemm_f32: shapes do not agree: %s %s -> %s" % (a.shape, b.shape, c.shape))
    with torch.cuda.device(c.device):
        rc = lib().ftb_bgemm_f32(a.data_ptr(), b.data_ptr(), c.data_ptr(), batch, m, n, k, int(trans_a),
                                 int(trans_b), _cfg_ptr(cfg), _status_ptr(status), _stream_ptr(stream))
    if rc:
        raise FtbError(rc, "ftb_bgemm_f32")


def bgemm_bf16(a, b, c, trans_a=False, trans_b=False, cfg=None, status=None, stream=None):
    """c[B,M,N] = op(a[b]) @ op(b[b]); bf16 inputs, fp32 accumulate, c bf16 or fp32."""
    _check(a, torch.bfloat16, "a")
    _check(b, torch.bfloat16, "b")
    if c.dtype not in (torch.bfloat16, torch.float32):
        raise TypeError("c must be bfloat16 or float32")
    _check(c, c.dtype, "c")
    batch, m, n = c.shape
    k = a.shape[1] if trans_a else a.shape[2]
    if (tuple(a.shape) != ((batch, k, m) if trans_a else (batch, m, k)) or
            tuple(b.shape) != ((batch, n, k) if trans_b else (batch, k, n))):
        raise ValueError("bgemm_bf16: shapes do not agree: %s %s -> %s" % (a.shape, b.shape, c.shape))
    with torch.cuda.device(c.device):
        rc = lib().ftb_bgemm_bf16(a.data_ptr(), b.data_ptr(), c.data_ptr(), batch, m, n, k, int(trans_a),
                                  int(trans_b), int(c.dtype == torch.float32), _cfg_ptr(cfg),
                                  _status_ptr(status), _stream_ptr(stream))
    if rc:
        raise FtbError(rc, "ftb_bgemm_bf16")


def bgemm_bf16_multi(a, b, dst_ptrs, m, n, trans_a=False, trans_b=False, out_f32=False, cfg=None, status=None,
                     stream=None):
    """Batched bf16 GEMM whose result goes to several buffers at once.

    ``dst_ptrs``: 1..8 device addresses (ints), each of a [batch, m, n] buffer on this GPU or a
    mapped buffer of a peer GPU (e.g. ``symm_mem`` buffer pointers plus the slice offset).
    """
    _check(a, torch.bfloat16, "a")
    _check(b, torch.bfloat16, "b")
    batch = a.shape[0]
    k = a.shape[1] if trans_a else a.shape[2]
    if (tuple(a.shape) != ((batch, k, m) if trans_a else (batch, m, k)) or
            tuple(b.shape) != ((batch, n, k) if trans_b else (batch, k, n))):
        raise ValueError("bgemm_bf16_multi: shapes do not agree: %s %s -> (%d, %d, %d)" % (a.shape, b.shape, batch, m, n))
    if not 1 <= len(dst_ptrs) <= 8:
        raise ValueError("between 1 and 8 destinations")
    arr = (ctypes.c_void_p * len(dst_ptrs))(*[ctypes.c_void_p(int(p)) for p in dst_ptrs])
    with torch.cuda.device(a.device):
        rc = lib().ftb_bgemm_bf16_multi(a.data_ptr(), b.data_ptr(), arr, len(dst_ptrs), batch, m, n, k,
                                        int(trans_a), int(trans_b), int(out_f32), _cfg_ptr(cfg),
                                        _status_ptr(status), _stream_ptr(stream))
    if rc:
        raise FtbError(rc, "ftb_bgemm_bf16_multi")


def gemm_s8(a, b, c, trans_a=False, trans_b=False, cfg=None, status=None, stream=None):
    """c[M,N] int32 = op(a) @ op(b) for int8 inputs, exact."""
    _check(a, torch.int8, "a")
    _check(b, torch.int8, "b")
    _check(c, torch.int32, "c")
    m, n = c.shape
    k = a.shape[0] if trans_a else a.shape[1]
    if tuple(a.shape) != ((k, m) if trans_a else (m, k)) or tuple(b.shape) != ((n, k) if trans_b else (k, n)):
        raise ValueError("gemm_s8: shapes do not agree: %s %s -> %s" % (a.shape, b.shape, c.shape))
    with torch.cuda.device(c.device):
        rc = lib().ftb_gemm_s8(a.data_ptr(), b.data_ptr(), c.data_ptr(), m, n, k, int(trans_a), int(trans_b),
                               _cfg_ptr(cfg), _status_ptr(status), _stream_ptr(stream))
    if rc:
        raise FtbError(rc, "ftb_gemm_s8")


def conv_out_size(size, kernel, stride, pad, dil):
    return (size + 2 * pad - dil * (kernel - 1) - 1) // stride + 1


def conv2d_workspace_bytes(n, c, h, w, k, r, s, groups=1):
    return int(lib().ftb_conv2d_workspace_bytes(n, c, h, w, k, r, s, groups))


def conv2d_pack_filter(weight, x_shape, stride=(1, 1), padding=(0, 0), dilation=(1, 1), groups=1, cfg=None,
                       workspace=None, stream=None):
    """Packs ``weight`` into the filter region of ``workspace`` for conv calls on inputs of
    ``x_shape`` with the same knobs; follow with ``conv2d_nchw_f32(..., prepacked=True)``."""
    _check(weight, torch.float32, "weight")
    n, c, h, w = (int(v) for v in x_shape)
    k, cg, r, s = weight.shape
    need = conv2d_workspace_bytes(n, c, h, w, k, r, s, groups)
    if workspace is None or workspace.numel() * workspace.element_size() < need:
        raise ValueError("conv2d: workspace of at least %d bytes required" % need)
    with torch.cuda.device(weight.device):
        rc = lib().ftb_conv2d_pack_filter(
            weight.data_ptr(), n, c, h, w, k, r, s, stride[0], stride[1], padding[0], padding[1], dilation[0],
            dilation[1], groups, _cfg_ptr(cfg), workspace.data_ptr(), workspace.numel() * workspace.element_size(),
            _stream_ptr(stream))
    if rc:
        raise FtbError(rc, "ftb_conv2d_pack_filter")


def conv2d_nchw_f32(x, weight, out, bias=None, stride=(1, 1), padding=(0, 0), dilation=(1, 1), groups=1,
                    cfg=None, workspace=None, status=None, stream=None, prepacked=False):
    """out[N,K,P,Q] = conv2d(x[N,C,H,W], weight[K,C/groups,R,S]) (+ bias); the caller owns
    ``workspace`` (a uint8 CUDA tensor of at least conv2d_workspace_bytes bytes).  ``prepacked``:
    the workspace already holds this weight's packing (``conv2d_pack_filter`` or an earlier call
    with the same shapes and knobs): only the input is laid out."""
    for t, nm in ((x, "x"), (weight, "weight"), (out, "out")):
        _check(t, torch.float32, nm)
    if bias is not None:
        _check(bias, torch.float32, "bias")
    n, c, h, w = x.shape
    k, cg, r, s = weight.shape
    if cg * groups != c:
        raise ValueError("conv2d: weight channels %d x groups %d != input channels %d" % (cg, groups, c))
    need = conv2d_workspace_bytes(n, c, h, w, k, r, s, groups)
    if workspace is None or workspace.numel() * workspace.element_size() < need:
        raise ValueError("conv2d: workspace of at least %d bytes required" % need)
    with torch.cuda.device(out.device):
        entry = lib().ftb_conv2d_nchw_f32_prepacked if prepacked else lib().ftb_conv2d_nchw_f32
        rc = entry(
            x.data_ptr(), weight.data_ptr(), bias.data_ptr() if bias is not None else None, out.data_ptr(),
            n, c, h, w, k, r, s, stride[0], stride[1], padding[0], padding[1], dilation[0], dilation[1],
            groups, _cfg_ptr(cfg), workspace.data_ptr(), workspace.numel() * workspace.element_size(),
            _status_ptr(status), _stream_ptr(stream))
    if rc:
        raise FtbError(rc, "ftb_conv2d_nchw_f32")


def conv2d_nchw_f32_multi(x, weight, dst_ptrs, bias=None, stride=(1, 1), padding=(0, 0), dilation=(1, 1), groups=1,
                          cfg=None, workspace=None, status=None, stream=None, prepacked=False):
    """conv2d whose result goes to several buffers at once (``dst_ptrs``: 1..8 device addresses of
    [N,K,P,Q] fp32 buffers, this GPU's or a peer's mapped memory).  Raises ``FtbError`` with code
    -2 when the kernel that serves the shape has a single destination."""
    for t, nm in ((x, "x"), (weight, "weight")):
        _check(t, torch.float32, nm)
    if bias is not None:
        _check(bias, torch.float32, "bias")
    n, c, h, w = x.shape
    k, cg, r, s = weight.shape
    if cg * groups != c:
        raise ValueError("conv2d: weight channels %d x groups %d != input channels %d" % (cg, groups, c))
    need = conv2d_workspace_bytes(n, c, h, w, k, r, s, groups)
    if workspace is None or workspace.numel() * workspace.element_size() < need:
        raise ValueError("conv2d: workspace of at least %d bytes required" % need)
    if not 1 <= len(dst_ptrs) <= 8:
        raise ValueError("between 1 and 8 destinations")
    arr = (ctypes.c_void_p * len(dst_ptrs))(*[ctypes.c_void_p(int(p)) for p in dst_ptrs])
    with torch.cuda.device(x.device):
        rc = lib().ftb_conv2d_nchw_f32_multi(
            x.data_ptr(), weight.data_ptr(), bias.data_ptr() if bias is not None else None, arr, len(dst_ptrs),
            n, c, h, w, k, r, s, stride[0], stride[1], padding[0], padding[1], dilation[0], dilation[1],
            groups, int(prepacked), _cfg_ptr(cfg), workspace.data_ptr(),
            workspace.numel() * workspace.element_size(), _status_ptr(status), _stream_ptr(stream))
    if rc:
        raise FtbError(rc, "ftb_conv2d_nchw_f32_multi")


def conv2d_nhwc_workspace_bytes(c, k, r, s, groups=1):
    return int(lib().ftb_conv2d_nhwc_workspace_bytes(c, k, r, s, groups))


def conv2d_nhwc_f32(x, weight, out, bias=None, stride=(1, 1), padding=(0, 0), dilation=(1, 1), groups=1,
                    cfg=None, workspace=None, status=None, stream=None, prepacked=False):
    """Channels-last conv2d: out[N,P,Q,K] = conv2d(x[N,H,W,C], weight[K,C/groups,R,S]) (+ bias), read and
    written where the tensors lie (no layout pass).  ``workspace``: a uint8 CUDA tensor of at least
    ``conv2d_nhwc_workspace_bytes`` bytes for the packed filter; ``prepacked``: it holds this weight's packing from an earlier call with the same shapes and knobs."""
    for t, nm in ((x, "x"), (weight, "weight"), (out, "out")):
        _check(t, torch.float32, nm)
    if bias is not None:
        _check(bias, torch.float32, "bias")
    n, h, w, c = x.shape
    k, cg, r, s = weight.shape
    if cg * groups != c:
        raise ValueError("conv2d: weight channels %d x groups %d != input channels %d" % (cg, groups, c))
    need = conv2d_nhwc_workspace_bytes(c, k, r, s, groups)
    if workspace is None or workspace.numel() * workspace.element_size() < need:
        raise ValueError("conv2d: workspace of at least %d bytes required" % need)
    with torch.cuda.device(out.device):
        rc = lib().ftb_conv2d_nhwc_f32(
            x.data_ptr(), weight.data_ptr(), bias.data_ptr() if bias is not None else None, out.data_ptr(),
            n, c, h, w, k, r, s, stride[0], stride[1], padding[0], padding[1], dilation[0], dilation[1],
            groups, int(prepacked), _cfg_ptr(cfg), workspace.data_ptr(),
            workspace.numel() * workspace.element_size(), _status_ptr(status), _stream_ptr(stream))
    if rc:
        raise FtbError(rc, "ftb_conv2d_nhwc_f32")


def _triple(value, what):
    if isinstance(value, int):
        return (value,) * 3
    value = tuple(int(v) for v in value)
    if len(value) != 3:
        raise ValueError("%s must be an int or three ints (depth, height, width)" % what)
    return value


def conv3d_workspace_bytes(n, c, d, h, w, k, t, r, s, groups=1):
    return int(lib().ftb_conv3d_workspace_bytes(n, c, d, h, w, k, t, r, s, groups))


def conv3d_ncdhw_f32(x, weight, out, bias=None, stride=1, padding=0, dilation=1, groups=1, cfg=None,
                     workspace=None, status=None, stream=None, prepacked=False):
    """out[N,K,OD,P,Q] = conv3d(x[N,C,D,H,W], weight[K,C/groups,T,R,S]) (+ bias); stride, padding and
    dilation are ints or (depth, height, width) triples.  The caller owns ``workspace`` (a uint8 CUDA
    tensor of at least conv3d_workspace_bytes bytes); ``prepacked``: it holds this weight's packing from an
    earlier call with the same shapes and knobs."""
    for t_, nm in ((x, "x"), (weight, "weight"), (out, "out")):
        _check(t_, torch.float32, nm)
    if bias is not None:
        _check(bias, torch.float32, "bias")
    n, c, d, h, w = x.shape
    k, cg, t, r, s = weight.shape
    if cg * groups != c:
        raise ValueError("conv3d: weight channels %d x groups %d != input channels %d" % (cg, groups, c))
    need = conv3d_workspace_bytes(n, c, d, h, w, k, t, r, s, groups)
    if workspace is None or workspace.numel() * workspace.element_size() < need:
        raise ValueError("conv3d: workspace of at least %d bytes required" % need)
    triple = ctypes.c_int32 * 3
    with torch.cuda.device(out.device):
        rc = lib().ftb_conv3d_ncdhw_f32(
            x.data_ptr(), weight.data_ptr(), bias.data_ptr() if bias is not None else None, out.data_ptr(),
            n, c, d, h, w, k, t, r, s, triple(*_triple(stride, "stride")), triple(*_triple(padding, "padding")),
            triple(*_triple(dilation, "dilation")), groups, int(prepacked), _cfg_ptr(cfg), workspace.data_ptr(),
            workspace.numel() * workspace.element_size(), _status_ptr(status), _stream_ptr(stream))
    if rc:
        raise FtbError(rc, "ftb_conv3d_ncdhw_f32")


NOALLOC_SCRATCH_BYTES = 8 * 1024 * 1024


def conv2d_nchw_f32_noalloc(x, weight, out, bias=None, stride=(1, 1), padding=(0, 0), dilation=(1, 1), groups=1,
                            cfg=None, status=None, stream=None):
    """conv2d for callers that may not allocate device memory (no workspace argument).

    Meant for code that is handed its buffers by another runtime, or runs where allocation is
    banned after start-up.  The workspace is a fixed 8 MiB array inside the library; shapes that
    need more raise ``FtbError`` with code -7.  Calls share that array: do not let two of them
    overlap on one GPU.  The first call on a device does a one-time address lookup and should
    happen before any stream capture begins.
    """
    for t, nm in ((x, "x"), (weight, "weight"), (out, "out")):
        _check(t, torch.float32, nm)
    if bias is not None:
        _check(bias, torch.float32, "bias")
    n, c, h, w = x.shape
    k, cg, r, s = weight.shape
    if cg * groups != c:
        raise ValueError("conv2d: weight channels %d x groups %d != input channels %d" % (cg, groups, c))
    with torch.cuda.device(out.device):
        rc = lib().ftb_conv2d_nchw_f32_noalloc(
            x.data_ptr(), weight.data_ptr(), bias.data_ptr() if bias is not None else None, out.data_ptr(),
            n, c, h, w, k, r, s, stride[0], stride[1], padding[0], padding[1], dilation[0], dilation[1],
            groups, _cfg_ptr(cfg), _status_ptr(status), _stream_ptr(stream))
    if rc:
        raise FtbError(rc, "ftb_conv2d_nchw_f32_noalloc")


def dwconv2d_nchw_f32(x, weight, out, bias=None, stride=(1, 1), padding=(0, 0), dilation=(1, 1), cfg=None,
                      status=None, stream=None):
    """out[N,C*f,P,Q] = depthwise conv of x[N,C,H,W] with weight[C,f,R,S] (+ bias)."""
    for t, nm in ((x, "x"), (weight, "weight"), (out, "out")):
        _check(t, torch.float32, nm)
    if bias is not None:
        _check(bias, torch.float32, "bias")
    n, c, h, w = x.shape
    c2, f, r, s = weight.shape
    if c2 != c:
        raise ValueError("depthwise: weight is [C,f,R,S] with C = input channels")
    with torch.cuda.device(out.device):
        rc = lib().ftb_dwconv2d_nchw_f32(
            x.data_ptr(), weight.data_ptr(), bias.data_ptr() if bias is not None else None, out.data_ptr(),
            n, c, h, w, f, r, s, stride[0], stride[1], padding[0], padding[1], dilation[0], dilation[1],
            _cfg_ptr(cfg), _status_ptr(status), _stream_ptr(stream))
    if rc:
        raise FtbError(rc, "ftb_dwconv2d_nchw_f32")


def dwconv2d_nchw_f32_multi(x, weight, dst_ptrs, bias=None, stride=(1, 1), padding=(0, 0), dilation=(1, 1), cfg=None,
                            status=None, stream=None):
    """Depthwise conv whose result goes to several buffers at once.

    ``dst_ptrs``: 1..8 device addresses (ints), each of an [N, C*f, P, Q] fp32 buffer on this GPU
    or a mapped buffer of a peer GPU (e.g. a rank's slice in every rank's gathered output).
    """
    for t, nm in ((x, "x"), (weight, "weight")):
        _check(t, torch.float32, nm)
    if bias is not None:
        _check(bias, torch.float32, "bias")
    n, c, h, w = x.shape
    c2, f, r, s = weight.shape
    if c2 != c:
        raise ValueError("depthwise: weight is [C,f,R,S] with C = input channels")
    if not 1 <= len(dst_ptrs) <= 8:
        raise ValueError("between 1 and 8 destinations")
    arr = (ctypes.c_void_p * len(dst_ptrs))(*[ctypes.c_void_p(int(p)) for p in dst_ptrs])
    with torch.cuda.device(x.device):
        rc = lib().ftb_dwconv2d_nchw_f32_multi(
            x.data_ptr(), weight.data_ptr(), bias.data_ptr() if bias is not None else None, arr, len(dst_ptrs),
            n, c, h, w, f, r, s, stride[0], stride[1], padding[0], padding[1], dilation[0], dilation[1],
            _cfg_ptr(cfg), _status_ptr(status), _stream_ptr(stream))
    if rc:
        raise FtbError(rc, "ftb_dwconv2d_nchw_f32_multi")
