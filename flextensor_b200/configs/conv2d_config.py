"""conv2d shape tables (reference: flextensor/configs/conv2d_config.py).

Every entry is the reference's 13-tuple
``(batch, in_channel, height, width, out_channel, _, k_h, k_w, _, stride, padding, dilation, groups)``
(layout documented at conv2d_config.py:19), generated here from compact per-network layer
lists ``(C, size, K, kernel, stride, pad[, groups])`` so that list positions, and with
them the task names "yolo3", "res5", ..., agree with the reference.
"""


def _expand(layers, batch=1):
    out = []
    for layer in layers:
        c, size, k, kernel, stride, pad = layer[:6]
        groups = layer[6] if len(layer) > 6 else 1
        out.append((batch, c, size, size, k, c, kernel, kernel, 1, stride, pad, 1, groups))
    return out


def copy_change_batch(batch, shape):
    return (batch,) + tuple(shape[1:])


_YOLO = [(3, 448, 64, 7, 2, 3), (64, 112, 192, 3, 1, 1), (192, 56, 128, 1, 1, 0), (128, 56, 256, 3, 1, 1),
         (256, 56, 256, 1, 1, 0), (256, 56, 512, 3, 1, 1), (512, 28, 256, 1, 1, 0), (256, 28, 512, 3, 1, 1),
         (512, 28, 512, 1, 1, 0), (512, 28, 1024, 3, 1, 1), (1024, 14, 512, 1, 1, 0), (512, 14, 1024, 3, 1, 1),
         (1024, 14, 1024, 3, 1, 1), (1024, 14, 1024, 3, 2, 1), (1024, 7, 1024, 3, 1, 1)]

# ResNet-50: stem, then per stage the distinct 1x1 / 3x3 / strided-1x1 convolutions
_RES = [(3, 224, 64, 7, 2, 3),
        (64, 56, 256, 1, 1, 0), (64, 56, 64, 1, 1, 0), (64, 56, 64, 3, 1, 1), (256, 56, 64, 1, 1, 0),
        (256, 56, 512, 1, 2, 0), (256, 56, 128, 1, 2, 0),
        (128, 28, 128, 3, 1, 1), (128, 28, 512, 1, 1, 0), (512, 28, 128, 1, 1, 0),
        (512, 28, 1024, 1, 2, 0), (512, 28, 256, 1, 2, 0),
        (256, 14, 256, 3, 1, 1), (256, 14, 1024, 1, 1, 0), (1024, 14, 256, 1, 1, 0),
        (1024, 14, 2048, 1, 2, 0), (1024, 14, 512, 1, 2, 0),
        (512, 7, 512, 3, 1, 1), (512, 7, 2048, 1, 1, 0), (2048, 7, 512, 1, 1, 0)]

_VGG16 = [(3, 224, 64, 3, 1, 1), (64, 224, 64, 3, 1, 1), (64, 112, 128, 3, 1, 1), (128, 112, 128, 3, 1, 1),
          (128, 56, 256, 3, 1, 1), (256, 56, 256, 3, 1, 1), (256, 28, 512, 3, 1, 1), (512, 28, 512, 3, 1, 1),
          (512, 14, 512, 3, 1, 1)]

_OVERFEAT = [(3, 192, 96, 11, 4, 5), (96, 24, 256, 5, 1, 2), (256, 12, 512, 3, 1, 1), (512, 12, 1024, 3, 1, 1),
             (1024, 12, 1024, 3, 1, 1)]

# MobileNet-v2 depthwise stages written as grouped convolutions (groups == C)
_MOBILEV2 = [(32, 112, 32, 3, 1, 1, 32), (16, 112, 96, 3, 2, 1, 16), (24, 56, 144, 3, 2, 1, 24),
             (32, 28, 192, 3, 2, 1, 32), (64, 14, 384, 3, 1, 1, 64), (96, 14, 576, 3, 2, 1, 96),
             (160, 7, 960, 3, 1, 1, 160)]


def _fire(c_in, size, squeeze, expand):
    return [(c_in, size, squeeze, 1, 1, 0), (squeeze, size, expand, 1, 1, 0), (squeeze, size, expand, 3, 1, 1)]


_SQUEEZE = ([(3, 227, 96, 7, 2, 0)] + _fire(96, 55, 16, 64) + [(128, 55, 16, 1, 1, 0)] + _fire(128, 55, 32, 128) +
            _fire(256, 27, 32, 128) + _fire(256, 27, 48, 192) + [(384, 27, 48, 1, 1, 0)] + _fire(384, 27, 64, 256) +
            _fire(512, 13, 64, 256) + [(512, 13, 1000, 1, 1, 0)])


# GoogLeNet: the reference lists each distinct layer shape once, hence the slices below
def _inception(c_in, size, b1, b3r, b3, b5r, b5, pool):
    return [(c_in, size, b1, 1, 1, 0), (c_in, size, b3r, 1, 1, 0), (b3r, size, b3, 3, 1, 1),
            (c_in, size, b5r, 1, 1, 0), (b5r, size, b5, 5, 1, 2), (c_in, size, pool, 1, 1, 0)]


_GOOGLE = ([(3, 224, 64, 7, 2, 3), (64, 56, 64, 1, 1, 0), (64, 56, 192, 3, 1, 1)] +
           _inception(192, 28, 64, 96, 128, 16, 32, 32) + _inception(256, 28, 128, 128, 192, 32, 96, 64)[1:] +
           _inception(480, 14, 192, 96, 208, 16, 48, 64) + _inception(512, 14, 160, 112, 224, 24, 64, 64) +
           _inception(512, 14, 128, 128, 256, 24, 64, 64)[1:3] +
           [(512, 14, 144, 1, 1, 0), (144, 14, 288, 3, 1, 1), (512, 14, 32, 1, 1, 0), (32, 14, 64, 5, 1, 2)] +
           _inception(528, 14, 256, 160, 320, 32, 128, 128) + _inception(832, 7, 256, 160, 320, 32, 128, 128) +
           _inception(832, 7, 384, 192, 384, 48, 128, 128)[0:5])

yolo_shapes_b1 = _expand(_YOLO)
yolo_shapes_b8 = [copy_change_batch(8, x) for x in yolo_shapes_b1]
yolo_shapes_b16 = [copy_change_batch(16, x) for x in yolo_shapes_b1]
yolo_shapes_b32 = [copy_change_batch(32, x) for x in yolo_shapes_b1]
yolo_shapes_b64 = [copy_change_batch(64, x) for x in yolo_shapes_b1]
yolo_shapes_b128 = [copy_change_batch(128, x) for x in yolo_shapes_b1]
yolo_shapes = yolo_shapes_b1

res_shapes_b1 = _expand(_RES)
res_shapes = [copy_change_batch(64, x) for x in res_shapes_b1]

vgg_16_shapes = _expand(_VGG16)
overfeat_shapes = _expand(_OVERFEAT)
mobilev2_shapes_b1 = _expand(_MOBILEV2)
mobilev2_shapes_b8 = [copy_change_batch(8, x) for x in mobilev2_shapes_b1]
mobilev2_shapes = mobilev2_shapes_b1
squeeze_shapes = _expand(_SQUEEZE)
google_shapes = _expand(_GOOGLE)

# the single entry of the reference's test table has zeros in the two unused fields
test_conv_shapes = [(256, 256, 14, 14, 512, 256, 1, 1, 0, 1, 0, 1, 1)]

# the ResNet-50 stage-2 3x3 layer at batch 1 (res_shapes_b1[3]) this backend is measured on
b200_conv2d_shape = res_shapes_b1[3]
