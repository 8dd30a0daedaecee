"""Grouped and dilated conv2d shape tables (reference: flextensor/configs/grouped_config.py:1-6 and
flextensor/configs/dilation_config.py:8-23), generated from compact rows.

Tuple layout: ``(batch, in_channel, H, W, out_channel, k, _, stride, padding, dilation, groups)``.
"""
# the 1x1 layer 1024 -> 512 at 14 x 14 split into 4, 8, 16 and 32 groups
grouped_shapes = [(1, 1024, 14, 14, 512, 1, 1, 1, 0, 1, g) for g in (4, 8, 16, 32)]

# YOLO layers from conv5 on, every filter dilated by 2: (C, size, K, kernel, stride, pad)
_DILATED = [(256, 56, 256, 1, 1, 0), (256, 56, 512, 3, 1, 1), (512, 28, 256, 1, 1, 0), (256, 28, 512, 3, 1, 1),
            (512, 28, 512, 1, 1, 0), (512, 28, 1024, 3, 1, 1), (1024, 14, 512, 1, 1, 0), (512, 14, 1024, 3, 1, 1),
            (1024, 14, 1024, 3, 1, 1), (1024, 14, 1024, 3, 2, 1), (1024, 7, 1024, 3, 1, 1)]
dilation_shapes = [(1, c, size, size, k, kernel, kernel, stride, pad, 2, 1) for c, size, k, kernel, stride, pad in _DILATED]
