"""Depthwise conv2d shape tables (reference: flextensor/configs/depthwise_config.py:1-31).

Tuple layout: ``(batch, in_channel, H, W, factor, k, _, stride, padding, dilation)``.
The MobileNet list is regenerated from ``(C, size, factor, stride)`` rows; the C = 256,
56 x 56 case this backend is measured on is not in the reference's tables and is
registered as an extra task.
"""
_MOBILE = [(32, 112, 1, 1), (16, 112, 6, 2), (24, 56, 6, 2), (32, 28, 6, 2), (64, 14, 6, 1), (96, 14, 6, 2),
           (160, 7, 6, 1)]


def _expand(batch):
    return [(batch, c, size, size, factor, 3, 3, stride, 1, 1) for c, size, factor, stride in _MOBILE]


depthwise_shapes = _expand(1)
depthwise_shapes_b8 = _expand(8)
depthwise_shapes_b16 = _expand(16)

b200_depthwise_shape = (1, 256, 56, 56, 1, 3, 3, 1, 1, 1)
