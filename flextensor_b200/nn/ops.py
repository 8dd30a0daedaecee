"""Compute definitions of the five hot-path operators, PyTorch conventions.

Each function returns the output ``Tensor`` of a small op graph (see ``ir.py``), with the
same argument meaning, shape checks, loop-axis names and output-size formulas as the
reference's ``flextensor/nn/ops.py``:

  zero_pad2d             ops.py:83-117
  conv2d_nchw            ops.py:419-479   (pad -> conv [-> bias]: a 2- or 3-op graph)
  depthwise_conv2d_nchw  ops.py:622-678   (weight layout [C, factor, kh, kw])
  conv2d_nhwc            ops.py:482-560   (conv2d_nchwc with one channel block: channels-last tensors)
  conv1d                 ops.py:293-351   (the same kernels, on a one-row image)
  zero_pad3d             ops.py:157-189
  conv3d_ncdhw           ops.py:689-751   (the per-tap conv kernel with a depth-tap loop)
  gemm_conv2d_nchw       ops.py:982-1044  (im2col -> GEMM -> col2img: the conv2d result by another route)
  conv2d_1x1_packed      task.py:168-173  (out[b,k,i] = sum_rc A[b,rc,i] * B[k,rc])
  gemm                   ops.py:1074-1108 (four transpose variants)
  batch_gemm             ops.py:1111-1158
  gemm_int8              no ops.py symbol; contract of test/test_tvm/legacy/gemm_int8.py:15-21

The reference is fp32 only; ``dtype`` follows the input tensors here so that the same
index expressions serve bf16 (fp32 accumulate) and int8 (int32 accumulate).
"""
from ..ir import ComputeOp, Tensor, reduce_axis
from ..utils import assert_print


def _pair(value, what):
    if isinstance(value, int):
        return (value, value)
    value = tuple(int(v) for v in value)
    assert_print(len(value) == 2, "%s must be an int or a pair" % what)
    return value


def _acc_dtype(dtype):
    return {"float32": "float32", "bfloat16": "float32", "int8": "int32"}.get(dtype, dtype)


def zero_pad2d(inputs, padding=0):
    """Zero padding of [batch, channel, height, width]; padding int, (h, w) or (up, down, left, right)."""
    if isinstance(padding, int):
        padding = (padding,) * 4
    assert_print(isinstance(padding, tuple), "type(padding)={}".format(type(padding)))
    if len(padding) == 2:
        padding = (padding[0], padding[0], padding[1], padding[1])
    assert_print(len(padding) == 4)
    b, c, h, w = (int(s) for s in inputs.shape)
    shape = (b, c, h + padding[0] + padding[1], w + padding[2] + padding[3])
    op = ComputeOp("pad2d", "Padding", shape, inputs.dtype, [inputs], ("b", "c", "h", "w"),
                   attrs={"padding": tuple(padding)})
    return op.output(0)


def _bias_add(output, bias):
    op = ComputeOp("bias_add", "bias_add", tuple(int(s) for s in output.shape), output.dtype,
                   [output, bias], ("b", "c", "h", "w"), attrs={"axis": 1})
    return op.output(0)


def relu(inputs):
    """max(x, 0) elementwise; following a convolution (or its bias) it is folded into the conv kernel's
    epilogue, as the bias is - the conv + bias + ReLU chain of a network runs as one kernel."""
    names = {3: ("b", "c", "l"), 5: ("b", "c", "d", "h", "w")}.get(len(inputs.shape), ("b", "c", "h", "w")[:len(inputs.shape)])
    op = ComputeOp("relu", "relu", tuple(int(s) for s in inputs.shape), inputs.dtype, [inputs], names)
    return op.output(0)


def conv2d_nchw(inputs, weight, bias=None, stride=1, padding=0, dilation=1, groups=1):
    """inputs [N,C,H,W], weight [K, C/groups, kh, kw] -> [N, K, out_h, out_w]."""
    n, c, in_h, in_w = (int(s) for s in inputs.shape)
    k, cg, k_h, k_w = (int(s) for s in weight.shape)
    assert_print(cg * groups == c)
    kg = k // groups
    assert_print(kg * groups == k)
    stride, padding, dilation = _pair(stride, "stride"), _pair(padding, "padding"), _pair(dilation, "dilation")
    out_h = (in_h + 2 * padding[0] - dilation[0] * (k_h - 1) - 1) // stride[0] + 1
    out_w = (in_w + 2 * padding[1] - dilation[1] * (k_w - 1) - 1) // stride[1] + 1
    rc = reduce_axis((0, cg), name="rc")
    rh = reduce_axis((0, k_h), name="rh")
    rw = reduce_axis((0, k_w), name="rw")
    padded = zero_pad2d(inputs, padding=padding)
    op = ComputeOp("conv2d", "compute", (n, k, out_h, out_w), _acc_dtype(inputs.dtype), [padded, weight],
                   ("b", "c", "h", "w"), reduce_axes=[rc, rw, rh],
                   attrs={"stride": stride, "padding": padding, "dilation": dilation, "groups": groups})
    out = op.output(0)
    if bias is not None:
        out = _bias_add(out, bias)
    return out


def conv2d_nhwc(inputs, weight, bias=None, stride=1, padding=0, dilation=1, groups=1):
    """inputs [N,H,W,C], weight [K, C/groups, kh, kw] -> [N, out_h, out_w, K]: the conv2d of ``conv2d_nchw`` on
    channels-last tensors.  The reference rewrites conv2d tasks to the blocked NCHWc layout for its CPU target
    (flextensor/nn/ops.py:482-560 conv2d_nchwc: [N, C/v, H, W, v]); with one block holding all channels that is
    this layout, which is the one the tensor-core kernels read without a layout pass."""
    n, in_h, in_w, c = (int(s) for s in inputs.shape)
    k, cg, k_h, k_w = (int(s) for s in weight.shape)
    assert_print(cg * groups == c)
    kg = k // groups
    assert_print(kg * groups == k)
    stride, padding, dilation = _pair(stride, "stride"), _pair(padding, "padding"), _pair(dilation, "dilation")
    out_h = (in_h + 2 * padding[0] - dilation[0] * (k_h - 1) - 1) // stride[0] + 1
    out_w = (in_w + 2 * padding[1] - dilation[1] * (k_w - 1) - 1) // stride[1] + 1
    rc = reduce_axis((0, cg), name="rc")
    rh = reduce_axis((0, k_h), name="rh")
    rw = reduce_axis((0, k_w), name="rw")
    pad_op = ComputeOp("pad2d", "Padding", (n, in_h + 2 * padding[0], in_w + 2 * padding[1], c), inputs.dtype, [inputs],
                       ("b", "h", "w", "c"), attrs={"padding": (padding[0], padding[0], padding[1], padding[1]),
                                                    "layout": "nhwc"})
    op = ComputeOp("conv2d", "compute", (n, out_h, out_w, k), _acc_dtype(inputs.dtype), [pad_op.output(0), weight],
                   ("b", "h", "w", "c"), reduce_axes=[rc, rw, rh],
                   attrs={"stride": stride, "padding": padding, "dilation": dilation, "groups": groups, "form": "nhwc"})
    out = op.output(0)
    if bias is not None:
        bop = ComputeOp("bias_add", "bias_add", (n, out_h, out_w, k), out.dtype, [out, bias], ("b", "h", "w", "c"),
                        attrs={"axis": 3})
        out = bop.output(0)
    return out


def zero_pad1d(inputs, padding=0):
    """Zero padding of [batch, channel, length]; padding int or (left, right)."""
    if isinstance(padding, int):
        padding = (padding, padding)
    assert_print(isinstance(padding, tuple) and len(padding) == 2, "type(padding)={}".format(type(padding)))
    b, c, l = (int(s) for s in inputs.shape)
    op = ComputeOp("pad2d", "Padding", (b, c, l + padding[0] + padding[1]), inputs.dtype, [inputs], ("b", "c", "l"),
                   attrs={"padding": tuple(padding)})
    return op.output(0)


def conv1d(inputs, weight, bias=None, stride=1, padding=0, dilation=1, groups=1):
    """inputs [N,C,L], weight [K, C/groups, k] -> [N, K, out_len]: served by the conv2d kernels
    on a one-row image (flextensor/nn/ops.py:293-351)."""
    n, c, in_len = (int(s) for s in inputs.shape)
    k, cg, k_len = (int(s) for s in weight.shape)
    assert_print(cg * groups == c, "left=%d, right=%d" % (cg * groups, c))
    assert_print(k % groups == 0)
    stride = stride[0] if isinstance(stride, tuple) else int(stride)
    padding = padding[0] if isinstance(padding, tuple) else int(padding)
    dilation = int(dilation)
    out_len = (in_len + 2 * padding - dilation * (k_len - 1) - 1) // stride + 1
    rc = reduce_axis((0, cg), name="rc")
    rl = reduce_axis((0, k_len), name="rl")
    padded = zero_pad1d(inputs, padding=padding)
    op = ComputeOp("conv2d", "compute", (n, k, out_len), _acc_dtype(inputs.dtype), [padded, weight],
                   ("b", "c", "l"), reduce_axes=[rc, rl],
                   attrs={"stride": (1, stride), "padding": (0, padding), "dilation": (1, dilation), "groups": groups,
                          "form": "conv1d"})
    out = op.output(0)
    if bias is not None:
        bop = ComputeOp("bias_add", "bias_add", (n, k, out_len), out.dtype, [out, bias], ("b", "c", "l"),
                        attrs={"axis": 1})
        out = bop.output(0)
    return out


def _triple(value, what):
    if isinstance(value, int):
        return (value, value, value)
    value = tuple(int(v) for v in value)
    assert_print(len(value) == 3, "%s must be an int or a triple" % what)
    return value


def zero_pad3d(inputs, padding=0):
    """Zero padding of [batch, channel, depth, height, width]; padding int, (d, h, w) or
    (d_up, d_down, h_up, h_down, w_up, w_down)."""
    if isinstance(padding, int):
        padding = (padding,) * 6
    assert_print(isinstance(padding, tuple), "type(padding)={}".format(type(padding)))
    if len(padding) == 3:
        padding = (padding[0], padding[0], padding[1], padding[1], padding[2], padding[2])
    assert_print(len(padding) == 6)
    b, c, d, h, w = (int(s) for s in inputs.shape)
    shape = (b, c, d + padding[0] + padding[1], h + padding[2] + padding[3], w + padding[4] + padding[5])
    op = ComputeOp("pad2d", "Padding", shape, inputs.dtype, [inputs], ("b", "c", "d", "h", "w"),
                   attrs={"padding": tuple(padding)})
    return op.output(0)


def conv3d_ncdhw(inputs, weight, bias=None, stride=1, padding=0, dilation=1, groups=1):
    """inputs [N,C,D,H,W], weight [K, C/groups, kd, kh, kw] -> [N, K, out_d, out_h, out_w]
    (flextensor/nn/ops.py:689-751)."""
    n, c, in_d, in_h, in_w = (int(s) for s in inputs.shape)
    k, cg, k_d, k_h, k_w = (int(s) for s in weight.shape)
    assert_print(cg * groups == c)
    kg = k // groups
    assert_print(kg * groups == k)
    stride, padding, dilation = _triple(stride, "stride"), _triple(padding, "padding"), _triple(dilation, "dilation")
    out_d = (in_d + 2 * padding[0] - dilation[0] * (k_d - 1) - 1) // stride[0] + 1
    out_h = (in_h + 2 * padding[1] - dilation[1] * (k_h - 1) - 1) // stride[1] + 1
    out_w = (in_w + 2 * padding[2] - dilation[2] * (k_w - 1) - 1) // stride[2] + 1
    rc = reduce_axis((0, cg), name="rc")
    rd = reduce_axis((0, k_d), name="rd")
    rh = reduce_axis((0, k_h), name="rh")
    rw = reduce_axis((0, k_w), name="rw")
    padded = zero_pad3d(inputs, padding=padding)
    op = ComputeOp("conv2d", "compute", (n, k, out_d, out_h, out_w), _acc_dtype(inputs.dtype), [padded, weight],
                   ("b", "c", "d", "h", "w"), reduce_axes=[rc, rd, rw, rh],
                   attrs={"stride": stride, "padding": padding, "dilation": dilation, "groups": groups,
                          "form": "conv3d"})
    out = op.output(0)
    if bias is not None:
        bop = ComputeOp("bias_add", "bias_add", (n, k, out_d, out_h, out_w), out.dtype, [out, bias],
                        ("b", "c", "d", "h", "w"), attrs={"axis": 1})
        out = bop.output(0)
    return out


def gemm_conv2d_nchw(inputs, weight, bias=None, stride=1, padding=0, dilation=1, groups=1):
    """The reference builds this result as im2col -> GEMM -> col2img (flextensor/nn/ops.py:982-1044);
    the numbers are those of ``conv2d_nchw``, and here the same implicit-GEMM kernels compute them
    without materialising the column matrix."""
    return conv2d_nchw(inputs, weight, bias=bias, stride=stride, padding=padding, dilation=dilation, groups=groups)


def conv2d_1x1_packed(A, B):
    """out[b,k,i] = sum_rc A[b,rc,i] * B[k,rc]: a 1x1 convolution on pixels packed into one axis
    (flextensor/task.py:168-173), i.e. a batched GEMM with the same left operand for every item."""
    n, c, hw = (int(s) for s in A.shape)
    k, c2 = (int(s) for s in B.shape)
    assert_print(c2 == c)
    rc = reduce_axis((0, c), name="rc")
    op = ComputeOp("conv2d", "compute", (n, k, hw), _acc_dtype(A.dtype), [A, B], ("b", "k", "i"), reduce_axes=[rc],
                   attrs={"stride": (1, 1), "padding": (0, 0), "dilation": (1, 1), "groups": 1, "form": "packed_1x1"})
    return op.output(0)


def depthwise_conv2d_nchw(inputs, weight, bias=None, stride=1, padding=0, dilation=1):
    """inputs [N,C,H,W], weight [C, factor, kh, kw] -> [N, C*factor, out_h, out_w]."""
    n, c, in_h, in_w = (int(s) for s in inputs.shape)
    c2, factor, k_h, k_w = (int(s) for s in weight.shape)
    assert_print(c2 == c)
    stride, padding, dilation = _pair(stride, "stride"), _pair(padding, "padding"), _pair(dilation, "dilation")
    out_h = (in_h + 2 * padding[0] - dilation[0] * (k_h - 1) - 1) // stride[0] + 1
    out_w = (in_w + 2 * padding[1] - dilation[1] * (k_w - 1) - 1) // stride[1] + 1
    rh = reduce_axis((0, k_h), name="rh")
    rw = reduce_axis((0, k_w), name="rw")
    padded = zero_pad2d(inputs, padding=padding)
    op = ComputeOp("depthwise_conv2d", "compute", (n, c * factor, out_h, out_w), _acc_dtype(inputs.dtype),
                   [padded, weight], ("b", "c", "h", "w"), reduce_axes=[rw, rh],
                   attrs={"stride": stride, "padding": padding, "dilation": dilation, "factor": factor})
    out = op.output(0)
    if bias is not None:
        out = _bias_add(out, bias)
    return out


def _gemm_dims(a_shape, b_shape, transposeA, transposeB):
    """(M, N, K) of op(A).op(B) for 2-d shapes, with the reference's shape assertion."""
    if transposeA and transposeB:      # A[k,i], B[j,k]
        assert_print(a_shape[0] == b_shape[1])
        return a_shape[1], b_shape[0], b_shape[1]
    if transposeA:                     # A[k,i], B[k,j]
        assert_print(a_shape[0] == b_shape[0])
        return a_shape[1], b_shape[1], b_shape[0]
    if transposeB:                     # A[i,k], B[j,k]
        assert_print(a_shape[1] == b_shape[1])
        return a_shape[0], b_shape[0], b_shape[1]
    assert_print(a_shape[1] == b_shape[0])  # A[i,k], B[k,j]
    return a_shape[0], b_shape[1], b_shape[0]


def gemm(A, B, transposeA=False, transposeB=False):
    """C[i,j] = sum_k op(A)[i,k] * op(B)[k,j]."""
    m, n, k = _gemm_dims([int(s) for s in A.shape], [int(s) for s in B.shape], transposeA, transposeB)
    rk = reduce_axis((0, k), name="k")
    op = ComputeOp("gemm", "compute", (m, n), _acc_dtype(A.dtype), [A, B], ("i", "j"), reduce_axes=[rk],
                   attrs={"transposeA": bool(transposeA), "transposeB": bool(transposeB)})
    return op.output(0)


def batch_gemm(A, B, transposeA=False, transposeB=False, out_dtype=None):
    """C[b,i,j] = sum_k op(A[b])[i,k] * op(B[b])[k,j]; ``out_dtype`` defaults to the input dtype
    for bf16 (accumulation is always fp32) and to fp32 for fp32."""
    a_shape, b_shape = [int(s) for s in A.shape], [int(s) for s in B.shape]
    assert_print(a_shape[0] == b_shape[0])
    m, n, k = _gemm_dims(a_shape[1:], b_shape[1:], transposeA, transposeB)
    rk = reduce_axis((0, k), name="k")
    dtype = out_dtype or A.dtype
    op = ComputeOp("batch_gemm", "compute", (a_shape[0], m, n), dtype, [A, B], ("b", "i", "j"),
                   reduce_axes=[rk], attrs={"transposeA": bool(transposeA), "transposeB": bool(transposeB)})
    return op.output(0)


def gemm_int8(A, B, transposeA=False, transposeB=False):
    """int8 x int8 -> int32 GEMM; ``transposeB=True`` is the legacy script's B[n,k] layout."""
    assert_print(A.dtype == "int8" and B.dtype == "int8", "gemm_int8 takes int8 tensors")
    m, n, k = _gemm_dims([int(s) for s in A.shape], [int(s) for s in B.shape], transposeA, transposeB)
    rk = reduce_axis((0, k), name="k")
    op = ComputeOp("gemm_int8", "compute", (m, n), "int32", [A, B], ("i", "j"), reduce_axes=[rk],
                   attrs={"transposeA": bool(transposeA), "transposeB": bool(transposeB)})
    return op.output(0)
