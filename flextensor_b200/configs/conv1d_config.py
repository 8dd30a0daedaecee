"""conv1d shape table (reference: flextensor/configs/conv1d_config.py): YOLO layers with the image
flattened to a sequence.  Tuple layout:
``(batch, in_channel, length, out_channel, _, k_len, _, stride, padding, dilation, groups)``.
"""
_ROWS = [(192, 56 * 56, 128, 1, 0), (128, 56 * 56, 256, 9, 1), (512, 28 * 28, 256, 1, 0), (256, 28 * 28, 512, 9, 1),
         (1024, 196, 512, 1, 0), (512, 196, 1024, 9, 1), (1024, 49, 1024, 9, 1)]
conv1d_shapes = [(1, c, length, k, c, k_len, 1, 1, pad, 1, 1) for c, length, k, k_len, pad in _ROWS]
