"""TEST INFRASTRUCTURE - ctypes loader of ``oracle/ft_oracle.c`` (see that file's header).

``build()`` runs the Makefile; ``lib()`` loads ``oracle/build/libft_oracle.so``.  The
wrappers take and return numpy arrays.
"""
import ctypes
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "build", "libft_oracle.so")
_lib = None


def build(force=False):
    src = os.path.join(HERE, "ft_oracle.c")
    if force or not os.path.exists(LIB) or os.path.getmtime(src) > os.path.getmtime(LIB):
        cmd = ["make", "-C", HERE] + (["-B"] if force else [])
        # -march=native code must be rebuilt on the machine that runs it
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError("oracle build failed:\n%s\n%s" % (proc.stdout, proc.stderr))
    return LIB


def lib():
    global _lib
    if _lib is None:
        build()
        try:
            _lib = ctypes.CDLL(LIB)
            _lib.fto_max_threads()
        except OSError:
            build(force=True)
            _lib = ctypes.CDLL(LIB)
        _lib.fto_max_threads.restype = ctypes.c_int
    return _lib


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p) if a is not None else None


def _i64(*vals):
    return [ctypes.c_int64(int(v)) for v in vals]


def _int(*vals):
    return [ctypes.c_int(int(v)) for v in vals]


def max_threads():
    return int(lib().fto_max_threads())


def use_all_cores():
    """Let the tiled nests use every core this process may run on; returns the thread count."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    lib().fto_set_threads(ctypes.c_int(n))
    return max_threads()


def gemm_f32_naive(a, b, ta=False, tb=False, acc64=True):
    m = a.shape[1] if ta else a.shape[0]
    k = a.shape[0] if ta else a.shape[1]
    n = b.shape[0] if tb else b.shape[1]
    c = np.empty((m, n), dtype=np.float32)
    lib().fto_gemm_f32_naive(_p(np.ascontiguousarray(a)), _p(np.ascontiguousarray(b)), _p(c), *_i64(m, n, k),
                             *_int(ta, tb, acc64))
    return c


def bgemm_bf16_naive(a_bits, b_bits, ta=False, tb=False, out_f32=False):
    batch = a_bits.shape[0]
    m = a_bits.shape[2] if ta else a_bits.shape[1]
    k = a_bits.shape[1] if ta else a_bits.shape[2]
    n = b_bits.shape[1] if tb else b_bits.shape[2]
    c = np.empty((batch, m, n), dtype=np.float32 if out_f32 else np.uint16)
    lib().fto_bgemm_bf16_naive(_p(np.ascontiguousarray(a_bits)), _p(np.ascontiguousarray(b_bits)), _p(c),
                               *_i64(batch, m, n, k), *_int(ta, tb, out_f32))
    return c


def gemm_s8_naive(a, b, ta=False, tb=False):
    m = a.shape[1] if ta else a.shape[0]
    k = a.shape[0] if ta else a.shape[1]
    n = b.shape[0] if tb else b.shape[1]
    c = np.empty((m, n), dtype=np.int32)
    lib().fto_gemm_s8_naive(_p(np.ascontiguousarray(a)), _p(np.ascontiguousarray(b)), _p(c), *_i64(m, n, k),
                            *_int(ta, tb))
    return c


def _out_size(size, kernel, stride, pad, dil):
    return (size + 2 * pad - dil * (kernel - 1) - 1) // stride + 1


def conv2d_naive(x, w, bias=None, stride=(1, 1), padding=(0, 0), dilation=(1, 1), groups=1, acc64=True):
    n, c, h, wd = x.shape
    k, _, r, s = w.shape
    p = _out_size(h, r, stride[0], padding[0], dilation[0])
    q = _out_size(wd, s, stride[1], padding[1], dilation[1])
    out = np.empty((n, k, p, q), dtype=np.float32)
    rc = lib().fto_conv2d_nchw_f32_naive(_p(np.ascontiguousarray(x)), _p(np.ascontiguousarray(w)),
                                         _p(np.ascontiguousarray(bias)) if bias is not None else None, _p(out),
                                         *_i64(n, c, h, wd, k, r, s, stride[0], stride[1], padding[0], padding[1],
                                               dilation[0], dilation[1], groups), *_int(acc64))
    assert rc == 0
    return out


def dwconv2d_naive(x, w, bias=None, stride=(1, 1), padding=(0, 0), dilation=(1, 1), acc64=True):
    n, c, h, wd = x.shape
    _, f, r, s = w.shape
    p = _out_size(h, r, stride[0], padding[0], dilation[0])
    q = _out_size(wd, s, stride[1], padding[1], dilation[1])
    out = np.empty((n, c * f, p, q), dtype=np.float32)
    rc = lib().fto_dwconv2d_nchw_f32_naive(_p(np.ascontiguousarray(x)), _p(np.ascontiguousarray(w)),
                                           _p(np.ascontiguousarray(bias)) if bias is not None else None, _p(out),
                                           *_i64(n, c, h, wd, f, r, s, stride[0], stride[1], padding[0], padding[1],
                                                 dilation[0], dilation[1]), *_int(acc64))
    assert rc == 0
    return out


# ---- llvm-template loop nests (timed CPU baseline); all OpenMP threads of the host
def gemm_f32_tiled(a, b, ti=8, tj=64, tk=64, out=None):
    m, k = a.shape
    n = b.shape[1]
    c = out if out is not None else np.empty((m, n), dtype=np.float32)
    lib().fto_gemm_f32_tiled(_p(a), _p(b), _p(c), *_i64(m, n, k), *_int(ti, tj, tk))
    return c


def bgemm_bf16_tiled(a_bits, b_bits, ti=8, tj=64, tk=64, out=None):
    batch, m, k = a_bits.shape
    n = b_bits.shape[2]
    c = out if out is not None else np.empty((batch, m, n), dtype=np.uint16)
    lib().fto_bgemm_bf16_tiled(_p(a_bits), _p(b_bits), _p(c), *_i64(batch, m, n, k), *_int(ti, tj, tk))
    return c


def gemm_s8_tiled(a, b, ti=8, tj=64, tk=64, out=None):
    m, k = a.shape
    n = b.shape[1]
    c = out if out is not None else np.empty((m, n), dtype=np.int32)
    lib().fto_gemm_s8_tiled(_p(a), _p(b), _p(c), *_i64(m, n, k), *_int(ti, tj, tk))
    return c


def conv2d_tiled(x, w, stride=(1, 1), padding=(0, 0), dilation=(1, 1), tk=4, out=None):
    n, c, h, wd = x.shape
    k, _, r, s = w.shape
    p = _out_size(h, r, stride[0], padding[0], dilation[0])
    q = _out_size(wd, s, stride[1], padding[1], dilation[1])
    o = out if out is not None else np.empty((n, k, p, q), dtype=np.float32)
    rc = lib().fto_conv2d_nchw_f32_tiled(_p(x), _p(w), _p(o), *_i64(n, c, h, wd, k, r, s, stride[0], stride[1],
                                                                     padding[0], padding[1], dilation[0], dilation[1]),
                                         *_int(tk))
    assert rc == 0
    return o


def dwconv2d_tiled(x, w, stride=(1, 1), padding=(0, 0), dilation=(1, 1), th=4, out=None):
    n, c, h, wd = x.shape
    _, f, r, s = w.shape
    p = _out_size(h, r, stride[0], padding[0], dilation[0])
    q = _out_size(wd, s, stride[1], padding[1], dilation[1])
    o = out if out is not None else np.empty((n, c * f, p, q), dtype=np.float32)
    rc = lib().fto_dwconv2d_nchw_f32_tiled(_p(x), _p(w), _p(o), *_i64(n, c, h, wd, f, r, s, stride[0], stride[1],
                                                                       padding[0], padding[1], dilation[0], dilation[1]),
                                           *_int(th))
    assert rc == 0
    return o
