"""conv3d shape table (reference: flextensor/configs/conv3d_config.py): the 3-D ResNet-18 layers after the
stem, batch 1.  Tuple layout as there:
``(batch, in_channel, depth, height, width, out_channel, _, kernel, _, stride, padding, dilation, groups)``.
"""
_ROWS = [
    # (in_channel, depth, height/width, out_channel, kernel, stride, padding)
    (64, 8, 28, 64, 3, 1, 1),                                # conv2_x
    (64, 8, 28, 128, 3, 2, 1), (128, 4, 14, 128, 3, 1, 1), (64, 8, 28, 128, 1, 2, 0),     # conv3_x
    (128, 4, 14, 256, 3, 2, 1), (256, 2, 7, 256, 3, 1, 1), (128, 4, 14, 256, 1, 2, 0),    # conv4_x
    (256, 2, 7, 512, 3, 2, 1), (512, 1, 3, 512, 3, 1, 1), (256, 2, 7, 512, 1, 2, 0),      # conv5_x
]
conv3d_shapes = [(1, c, d, hw, hw, k, c, ks, 1, st, pad, 1, 1) for c, d, hw, k, ks, st, pad in _ROWS]
