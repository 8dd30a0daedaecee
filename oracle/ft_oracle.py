"""TEST INFRASTRUCTURE - numpy restatement of the reference's compute definitions.

Each function follows the index expression of the reference operator it names, in
``flextensor/nn/ops.py`` of pku-liang/FlexTensor:

  zero_pad2d             ops.py:83-117   P[b,c,h,w] = in[b,c,h-p0,w-p2] inside, else 0
  conv2d_nchw            ops.py:419-479  out[b,k,h,w] = sum_{rc,rw,rh} P[b,(k//Kg)*Cg+rc, h*s+rh*d, w*s+rw*d] * W[k,rc,rh,rw]
                                         out_h = (H + 2p - d(kh-1) - 1)//s + 1, optional + bias[k]
  depthwise_conv2d_nchw  ops.py:622-678  out[b,c,h,w] = sum_{rw,rh} P[b,c//f, h*s+rh*d, w*s+rw*d] * W[c//f, c%f, rh, rw]
  gemm                   ops.py:1074-1108 (four transpose variants)
  batch_gemm             ops.py:1111-1158
  gemm_int8              flextensor/test/test_tvm/legacy/gemm_int8.py:15-21,143-148 (int32 accumulation, checked
                         against np.dot on int32 there)

Pinning: the reference's own tests hold no golden vectors; they compare conv2d and
depthwise against torch CPU on random inputs (flextensor/test/test_ops.py:85-115,
152-184).  ``tests/test_oracle.py`` repeats exactly those comparisons (same shapes,
strides, groups and tolerances) against this restatement, and checks it against the
committed fixtures of ``tests/golden``.  gemm, batch_gemm and int8 GEMM have no test in
the reference: for those three, parity is unpinned beyond the mathematical definition.

Accumulation: ``acc="f64"`` (default) accumulates in float64 and is the "truth" the GPU
results are judged against; ``acc="f32"`` mimics an fp32 implementation.
"""
import numpy as np


def _pair(v):
    return (int(v), int(v)) if np.isscalar(v) else (int(v[0]), int(v[1]))


def out_size(size, kernel, stride, pad, dil):
    return (size + 2 * pad - dil * (kernel - 1) - 1) // stride + 1


def zero_pad2d(x, padding=0):
    if np.isscalar(padding):
        padding = (padding,) * 4
    padding = tuple(int(p) for p in padding)
    if len(padding) == 2:
        padding = (padding[0], padding[0], padding[1], padding[1])
    assert len(padding) == 4
    b, c, h, w = x.shape
    out = np.zeros((b, c, h + padding[0] + padding[1], w + padding[2] + padding[3]), dtype=x.dtype)
    out[:, :, padding[0]:padding[0] + h, padding[2]:padding[2] + w] = x
    return out


def _acc_dtype(acc):
    return {"f64": np.float64, "f32": np.float32}[acc]


def conv2d_nchw(x, weight, bias=None, stride=1, padding=0, dilation=1, groups=1, acc="f64", out_dtype=np.float32):
    stride, padding, dilation = _pair(stride), _pair(padding), _pair(dilation)
    n, c, h, w = x.shape
    k, cg, kh, kw = weight.shape
    assert cg * groups == c and k % groups == 0
    kg = k // groups
    oh = out_size(h, kh, stride[0], padding[0], dilation[0])
    ow = out_size(w, kw, stride[1], padding[1], dilation[1])
    at = _acc_dtype(acc)
    padded = zero_pad2d(x, padding).astype(at)
    wt = weight.astype(at)
    out = np.zeros((n, k, oh, ow), dtype=at)
    for g in range(groups):
        pg = padded[:, g * cg:(g + 1) * cg]
        wg = wt[g * kg:(g + 1) * kg]
        for rh in range(kh):
            for rw in range(kw):
                h0, w0 = rh * dilation[0], rw * dilation[1]
                win = pg[:, :, h0:h0 + (oh - 1) * stride[0] + 1:stride[0], w0:w0 + (ow - 1) * stride[1] + 1:stride[1]]
                # out[b,k,h,w] += sum_rc win[b,rc,h,w] * W[k,rc,rh,rw]
                out[:, g * kg:(g + 1) * kg] += np.einsum("bchw,kc->bkhw", win, wg[:, :, rh, rw], optimize=True)
    if bias is not None:
        out += bias.astype(at).reshape(1, k, 1, 1)
    return out.astype(out_dtype)


def conv1d(x, weight, bias=None, stride=1, padding=0, dilation=1, groups=1, acc="f64", out_dtype=np.float32):
    """out[b,c,l] = sum_{rc,rl} padded[b, c//Kg*Cg + rc, l*stride + rl*dilation] * weight[c,rc,rl]
    (flextensor/nn/ops.py:339-347): the 2-d expression with one image row."""
    n, c, length = x.shape
    k, cg, k_len = weight.shape
    out = conv2d_nchw(x.reshape(n, c, 1, length), weight.reshape(k, cg, 1, k_len), bias, (1, stride), (0, padding),
                      (1, dilation), groups, acc=acc, out_dtype=out_dtype)
    return out.reshape(n, k, -1)


def conv3d_ncdhw(x, weight, bias=None, stride=1, padding=0, dilation=1, groups=1, acc="f64", out_dtype=np.float32):
    """out[b,c,d,h,w] = sum_{rc,rd,rh,rw} padded[b, c//Kg*Cg + rc, d*sd + rd*dd, h*sh + rh*dh, w*sw + rw*dw]
    * weight[c,rc,rd,rh,rw] (+ bias[c]) (flextensor/nn/ops.py:157-189 zero_pad3d, :689-751 conv3d_ncdhw)."""
    def triple(v):
        return (v, v, v) if isinstance(v, int) else tuple(int(i) for i in v)
    stride, padding, dilation = triple(stride), triple(padding), triple(dilation)
    n, c, d, h, w = x.shape
    k, cg, kd, kh, kw = weight.shape
    assert cg * groups == c and k % groups == 0
    kg = k // groups
    od = out_size(d, kd, stride[0], padding[0], dilation[0])
    oh = out_size(h, kh, stride[1], padding[1], dilation[1])
    ow = out_size(w, kw, stride[2], padding[2], dilation[2])
    at = _acc_dtype(acc)
    padded = np.pad(x.astype(at), ((0, 0), (0, 0), (padding[0],) * 2, (padding[1],) * 2, (padding[2],) * 2))
    wt = weight.astype(at)
    out = np.zeros((n, k, od, oh, ow), dtype=at)
    for g in range(groups):
        pg = padded[:, g * cg:(g + 1) * cg]
        wg = wt[g * kg:(g + 1) * kg]
        for rd in range(kd):
            for rh in range(kh):
                for rw in range(kw):
                    d0, h0, w0 = rd * dilation[0], rh * dilation[1], rw * dilation[2]
                    win = pg[:, :, d0:d0 + (od - 1) * stride[0] + 1:stride[0],
                             h0:h0 + (oh - 1) * stride[1] + 1:stride[1], w0:w0 + (ow - 1) * stride[2] + 1:stride[2]]
                    out[:, g * kg:(g + 1) * kg] += np.einsum("bcdhw,kc->bkdhw", win, wg[:, :, rd, rh, rw], optimize=True)
    if bias is not None:
        out += bias.astype(at).reshape(1, k, 1, 1, 1)
    return out.astype(out_dtype)


def conv2d_1x1_packed(a, b, acc="f64", out_dtype=np.float32):
    """out[b,k,i] = sum_rc A[b,rc,i] * B[k,rc] (flextensor/task.py:168-173)."""
    at = _acc_dtype(acc)
    return np.einsum("bci,kc->bki", a.astype(at), b.astype(at), optimize=True).astype(out_dtype)


def depthwise_conv2d_nchw(x, weight, bias=None, stride=1, padding=0, dilation=1, acc="f64", out_dtype=np.float32):
    stride, padding, dilation = _pair(stride), _pair(padding), _pair(dilation)
    n, c, h, w = x.shape
    c2, f, kh, kw = weight.shape
    assert c2 == c
    oh = out_size(h, kh, stride[0], padding[0], dilation[0])
    ow = out_size(w, kw, stride[1], padding[1], dilation[1])
    at = _acc_dtype(acc)
    padded = zero_pad2d(x, padding).astype(at)
    wt = weight.astype(at)
    out = np.zeros((n, c, f, oh, ow), dtype=at)  # output channel co = c*f + m  <->  (c, m) = (co//f, co%f)
    for rh in range(kh):
        for rw in range(kw):
            h0, w0 = rh * dilation[0], rw * dilation[1]
            win = padded[:, :, h0:h0 + (oh - 1) * stride[0] + 1:stride[0], w0:w0 + (ow - 1) * stride[1] + 1:stride[1]]
            out += win[:, :, None, :, :] * wt[None, :, :, rh, rw, None, None]
    out = out.reshape(n, c * f, oh, ow)
    if bias is not None:
        out += bias.astype(at).reshape(1, c * f, 1, 1)
    return out.astype(out_dtype)


def _op(m, transpose):
    return np.swapaxes(m, -1, -2) if transpose else m


def gemm(a, b, transposeA=False, transposeB=False, acc="f64", out_dtype=np.float32):
    at = _acc_dtype(acc)
    return (_op(a, transposeA).astype(at) @ _op(b, transposeB).astype(at)).astype(out_dtype)


def batch_gemm(a, b, transposeA=False, transposeB=False, acc="f64", out_dtype=np.float32):
    assert a.shape[0] == b.shape[0]
    at = _acc_dtype(acc)
    return np.matmul(_op(a, transposeA).astype(at), _op(b, transposeB).astype(at)).astype(out_dtype)


def gemm_int8(a, b, transposeA=False, transposeB=False):
    """Exact int32 result.  float64 matmul is exact here: |sum| <= 127*127*K < 2^53 for any
    K this library accepts, and it is BLAS-backed where an int32 matmul is not."""
    assert a.dtype == np.int8 and b.dtype == np.int8
    out = _op(a, transposeA).astype(np.float64) @ _op(b, transposeB).astype(np.float64)
    return np.rint(out).astype(np.int64).astype(np.int32)


def gemm_int8_direct(a, b, transposeA=False, transposeB=False):
    """The same by literal int32 arithmetic (small shapes; cross-checks the float64 route)."""
    return _op(a, transposeA).astype(np.int32) @ _op(b, transposeB).astype(np.int32)


# ---------------------------------------------------------------- bf16 helpers
def to_bf16_bits(x):
    """float32 -> bfloat16 bit pattern (uint16), round to nearest even."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    rounding = ((u >> 16) & 1) + np.uint32(0x7FFF)
    return ((u + rounding) >> 16).astype(np.uint16)


def from_bf16_bits(bits):
    return (bits.astype(np.uint32) << 16).view(np.float32)


def round_to_bf16(x):
    """float32 values rounded to the nearest bfloat16, returned as float32."""
    return from_bf16_bits(to_bf16_bits(x))


# ---------------------------------------------------------------- seeded synthetic inputs
def _rng(seed):
    return np.random.Generator(np.random.PCG64(seed))


def gemm_inputs(m, n, k, seed=0):
    """uniform[-1,1) fp32 A[m,k], B[k,n]."""
    g = _rng(seed)
    return (g.uniform(-1, 1, (m, k)).astype(np.float32), g.uniform(-1, 1, (k, n)).astype(np.float32))


def conv2d_inputs(n, c, h, w, k, r, s, groups=1, seed=1):
    """normal(0,1) fp32 input and weights."""
    g = _rng(seed)
    return (g.standard_normal((n, c, h, w)).astype(np.float32),
            g.standard_normal((k, c // groups, r, s)).astype(np.float32))


def depthwise_inputs(n, c, h, w, f, r, s, seed=2):
    """uniform[-1,1) fp32 input and [C,f,R,S] weights."""
    g = _rng(seed)
    return (g.uniform(-1, 1, (n, c, h, w)).astype(np.float32), g.uniform(-1, 1, (c, f, r, s)).astype(np.float32))


def batch_gemm_item(index, m, n, k, seed=3, std=0.02):
    """Batch item ``index``: normal(0, std) rounded to bf16 (returned as float32 values).  The
    per-item seed makes a shard identical for any number of GPUs."""
    g = _rng(seed * 1_000_003 + index)
    a = round_to_bf16((g.standard_normal((m, k)) * std).astype(np.float32))
    b = round_to_bf16((g.standard_normal((k, n)) * std).astype(np.float32))
    return a, b


def gemm_int8_inputs(m, n, k, seed=4):
    """integers uniform in [-127, 127]."""
    g = _rng(seed)
    return (g.integers(-127, 128, (m, k), dtype=np.int8), g.integers(-127, 128, (k, n), dtype=np.int8))


# ---------------------------------------------------------------- tolerances (one place, used by every test)
def normalised_error(x, y):
    """max |x - y| / max(|y|, rms(y)) element-wise: relative error with an rms floor."""
    x = np.asarray(x, dtype=np.float64)
    y = np.asarray(y, dtype=np.float64)
    rms = np.sqrt(np.mean(y * y)) if y.size else 0.0
    denom = np.maximum(np.abs(y), max(rms, 1e-300))
    return float(np.max(np.abs(x - y) / denom)) if y.size else 0.0


TOLERANCE = {
    "gemm_f32_3xtf32": 1e-4,   # GEMM fp32 must match within 1e-4 relative (rms floor)
    "gemm_f32_tf32": 5e-3,     # single-pass TF32, reported separately
    "conv2d_tf32": 5e-3,       # reference's own conv tolerances are 1e-2 (test_ops.py:111) and 1e-3 (common.py:43)
    "conv2d_3xtf32": 1e-4,
    "depthwise_f32": 1e-5,     # 9-term fp32 sums
    "bgemm_bf16_out_f32": 1e-5,
}


def bf16_output_ok(x, y):
    """|x - y| <= 2^-7 |y| + 2^-8 rms(y): one bf16 rounding of an exact-product fp32 sum."""
    x = np.asarray(x, dtype=np.float64)
    y = np.asarray(y, dtype=np.float64)
    rms = np.sqrt(np.mean(y * y))
    return bool(np.all(np.abs(x - y) <= 2.0 ** -7 * np.abs(y) + 2.0 ** -8 * rms))
