"""Task registry: a task binds a compute-definition builder to concrete arguments.

Same surface as the reference's ``flextensor/task.py``: ``Task`` with the key format
``"{category}_{name}_{args}_{target}({dev_id})"`` (task.py:32-46), ``register_task`` /
``register`` with silent overwrite (task.py:49-57), ``TASK_TABLE`` (task.py:29), and the
per-operator builders that return ``([output.op], [inputs..., output])``: ``conv2d``
(task.py:74-78), ``depthwise_conv2d`` (task.py:96-100), ``gemm`` (task.py:145-149).
``batch_gemm`` and ``gemm_int8`` have no builder in the reference and are added in the
same style.  Every shape of the reference's tables for these operators is registered for
targets "llvm" (baseline harness only) and "cuda", devices 0-7 (the reference stops at 3;
the measurement pool of an 8-GPU box pins one task per device).
"""
from .configs.conv2d_config import (yolo_shapes, res_shapes, res_shapes_b1, google_shapes, squeeze_shapes,
                                    vgg_16_shapes, test_conv_shapes, yolo_shapes_b8, mobilev2_shapes,
                                    overfeat_shapes, b200_conv2d_shape)
from .configs.depthwise_config import depthwise_shapes, depthwise_shapes_b8, depthwise_shapes_b16, b200_depthwise_shape
from .configs.grouped_config import grouped_shapes, dilation_shapes
from .configs.conv1d_config import conv1d_shapes
from .configs.conv3d_config import conv3d_shapes
from .configs.gemm_config import gemm_shapes, test_gemm_shapes, b200_batch_gemm_shapes, b200_gemm_int8_shapes
from .ir import placeholder
from .nn import conv2d_nchw, depthwise_conv2d_nchw, gemm as op_gemm, batch_gemm as op_batch_gemm, \
    gemm_int8 as op_gemm_int8, conv1d as op_conv1d, gemm_conv2d_nchw, conv2d_1x1_packed as op_1x1_packed, conv3d_ncdhw, \
    conv2d_nhwc
from .space import EnumSpace

TASK_TABLE = {}
NUM_DEVICES = 8


class Task(object):
    def __init__(self, category, name, func, args, target, dev_id=0):
        self.key = "{}_{}_{}_{}({})".format(category, name, args, target, dev_id)
        self.name = name
        self.func = func
        self.args = args
        self.target = target
        self.dev_id = dev_id
        self.category = category
        self.special_space = {}

    def set_specific_space(self, key, type, knobs):
        if type == "enum":
            self.special_space[key] = EnumSpace(knobs)
        else:
            raise RuntimeError("Not supported space type: %s" % type)


def register_task(task, override=False):
    # as in the reference, a repeated key silently replaces the earlier task
    TASK_TABLE[task.key] = task


def register(func, category, name, args, target, dev_id=0, override=False):
    register_task(Task(category, name, func, args, target, dev_id), override=override)


# ---------------------------------------------------------------- builders
def conv2d(N, C, H, W, K, kernel_size, stride=1, padding=0, dilation=1, groups=1):
    Img = placeholder((N, C, H, W))
    Wt = placeholder((K, C // groups, kernel_size, kernel_size))
    Output = conv2d_nchw(Img, Wt, stride=stride, padding=padding, dilation=dilation, groups=groups)
    return [Output.op], [Img, Wt, Output]


def conv2d_nhwc_layout(N, C, H, W, K, kernel_size, stride=1, padding=0, dilation=1, groups=1):
    """The conv2d task on channels-last tensors, same arguments as ``conv2d`` (what the reference's
    conv2d_nchwc_layout, task.py:81-93, is to its CPU target: the layout its kernels want)."""
    Img = placeholder((N, H, W, C))
    Wt = placeholder((K, C // groups, kernel_size, kernel_size))
    Output = conv2d_nhwc(Img, Wt, stride=stride, padding=padding, dilation=dilation, groups=groups)
    return [Output.op], [Img, Wt, Output]


def conv1d(N, C, L, K, kernel, stride=1, padding=0, dilation=1, groups=1):
    Seq = placeholder((N, C, L))
    Wt = placeholder((K, C // groups, kernel))
    Output = op_conv1d(Seq, Wt, stride=stride, padding=padding, dilation=dilation, groups=groups)
    return [Output.op], [Seq, Wt, Output]


def conv3d(N, C, D, H, W, K, kernel_size, stride=1, padding=0, dilation=1, groups=1):
    Img = placeholder((N, C, D, H, W))
    Wt = placeholder((K, C // groups, kernel_size, kernel_size, kernel_size))
    Output = conv3d_ncdhw(Img, Wt, stride=stride, padding=padding, dilation=dilation, groups=groups)
    return [Output.op], [Img, Wt, Output]


def gemm_conv2d(N, C, H, W, K, kernel_size, stride=1, padding=0, dilation=1, groups=1):
    Img = placeholder((N, C, H, W))
    Wt = placeholder((K, C // groups, kernel_size, kernel_size))
    Output = gemm_conv2d_nchw(Img, Wt, stride=stride, padding=padding, dilation=dilation, groups=groups)
    return [Output.op], [Img, Wt, Output]


def conv2d_1x1_packed(N, C, H, W, K, kernel_size):
    A = placeholder((N, C, H * W))
    B = placeholder((K, C))
    Output = op_1x1_packed(A, B)
    return [Output.op], [A, B, Output]


def depthwise_conv2d(N, C, H, W, factor, kernel_size, stride=1, padding=0, dilation=1):
    Img = placeholder((N, C, H, W))
    Wt = placeholder((C, factor, kernel_size, kernel_size))
    Output = depthwise_conv2d_nchw(Img, Wt, stride=stride, padding=padding, dilation=dilation)
    return [Output.op], [Img, Wt, Output]


def gemm(N, K, M):
    A = placeholder((N, K))
    B = placeholder((K, M))
    Output = op_gemm(A, B)
    return [Output.op], [A, B, Output]


def batch_gemm(B, N, K, M, dtype="bfloat16"):
    """C[b] = A[b] (N x K) . B[b] (K x M); bf16 storage with fp32 accumulation by default."""
    A = placeholder((B, N, K), dtype=dtype)
    Bm = placeholder((B, K, M), dtype=dtype)
    Output = op_batch_gemm(A, Bm)
    return [Output.op], [A, Bm, Output]


def gemm_int8(N, K, M, transposeB=False):
    """int32 C = A (N x K, int8) . B (K x M, int8); ``transposeB`` stores B as [M, K]."""
    A = placeholder((N, K), dtype="int8")
    B = placeholder((M, K) if transposeB else (K, M), dtype="int8")
    Output = op_gemm_int8(A, B, transposeB=transposeB)
    return [Output.op], [A, B, Output]


# ---------------------------------------------------------------- registrations
def _register_all(category, name, func, args, targets=("llvm", "cuda")):
    for dev in range(NUM_DEVICES):
        for target in targets:
            register_task(Task(category, name, func, args, target, dev))


conv2d_shape_dict = {
    "yolo": yolo_shapes,
    "google": google_shapes,
    "res": res_shapes,
    "squeeze": squeeze_shapes,
    "vgg-16": vgg_16_shapes,
    "test": test_conv_shapes,
    "yolo_b8": yolo_shapes_b8,
    "mobile_v2": mobilev2_shapes,
    "overfeat": overfeat_shapes,
    "res_b1": res_shapes_b1,      # batch-1 ResNet-50 layers (res_b13 is the stage-2 3x3 conv)
}

for _name, _shapes in conv2d_shape_dict.items():
    for _i, _shape in enumerate(_shapes):
        _b, _c, _h, _w, _k, _, _kh, _kw, _, _st, _pad, _dil, _grp = _shape
        _register_all("conv2d", _name + str(_i), conv2d, (_b, _c, _h, _w, _k, _kh, _st, _pad, _dil, _grp))

# the same layer lists through the im2col -> GEMM -> col2img definition (task.py:346-363 registers them
# for every conv2d table; the batch-1 YOLO and ResNet lists are kept here)
for _name in ("yolo", "res_b1"):
    for _i, _shape in enumerate(conv2d_shape_dict[_name]):
        _b, _c, _h, _w, _k, _, _kh, _kw, _, _st, _pad, _dil, _grp = _shape
        _register_all("gemm_conv2d", _name + str(_i), gemm_conv2d, (_b, _c, _h, _w, _k, _kh, _st, _pad, _dil, _grp))

for _shape in grouped_shapes:
    _b, _c, _h, _w, _k, _kh, _, _st, _pad, _dil, _grp = _shape
    _register_all("conv2d", "grouped", conv2d, (_b, _c, _h, _w, _k, _kh, _st, _pad, _dil, _grp))

for _shape in dilation_shapes:
    _b, _c, _h, _w, _k, _kh, _, _st, _pad, _dil, _grp = _shape
    _register_all("conv2d", "dilation", conv2d, (_b, _c, _h, _w, _k, _kh, _st, _pad, _dil, _grp))

for _shape in conv1d_shapes:
    _b, _c, _l, _k, _, _kl, _, _st, _pad, _dil, _grp = _shape
    _register_all("conv1d", "conv1d", conv1d, (_b, _c, _l, _k, _kl, _st, _pad, _dil, _grp))

for _shape in conv3d_shapes:
    _b, _c, _d, _h, _w, _k, _, _ks, _, _st, _pad, _dil, _grp = _shape
    _register_all("conv3d", "conv3d", conv3d, (_b, _c, _d, _h, _w, _k, _ks, _st, _pad, _dil, _grp))

# the packed 1x1 convolution (task.py:218 registers this one shape)
_register_all("conv2d", "1x1-packed", conv2d_1x1_packed, (256, 256, 14, 14, 512, 1))

for _shape in list(depthwise_shapes) + list(depthwise_shapes_b8) + list(depthwise_shapes_b16) + [b200_depthwise_shape]:
    _b, _c, _h, _w, _f, _k, _, _st, _pad, _dil = _shape
    _register_all("conv2d", "depthwise", depthwise_conv2d, (_b, _c, _h, _w, _f, _k, _st, _pad, _dil))

for _shape in gemm_shapes:
    _n, _k, _m = _shape
    _register_all("gemm", "gemm", gemm, (_n, _k, _m))

for _shape in list(test_gemm_shapes) + list(b200_batch_gemm_shapes):
    _register_all("gemm", "batch_gemm", batch_gemm, tuple(_shape))

for _shape in b200_gemm_int8_shapes:
    _register_all("gemm", "gemm_int8", gemm_int8, tuple(_shape))
