"""conv2d driver (flextensor/optimize/optimize_conv2d.py:29-83): trial budgets are split
``[trials // 10, trials]`` between the padding stage and the conv stage (:55)."""
from ..configs.conv2d_config import res_shapes_b1, yolo_shapes_b1
from ..task import conv2d
from .driver import main

shapes = [res_shapes_b1[3]] + list(yolo_shapes_b1)


def args_of(shape):
    batch, in_channel, height, width, out_channel, _, k_h, k_w, _, stride, padding, dilation, groups = shape
    return (batch, in_channel, height, width, out_channel, k_h, stride, padding, dilation, groups)


if __name__ == "__main__":
    main("conv2d", "conv2d", conv2d, shapes, args_of, trials_of=lambda t: [max(t // 10, 1), t])
