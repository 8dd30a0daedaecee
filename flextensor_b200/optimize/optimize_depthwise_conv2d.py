"""Depthwise conv2d driver (flextensor/optimize/optimize_depthwise_conv2d.py:18-71)."""
from ..configs.depthwise_config import b200_depthwise_shape, depthwise_shapes
from ..task import depthwise_conv2d
from .driver import main

shapes = [b200_depthwise_shape] + list(depthwise_shapes)


def args_of(shape):
    batch, in_channel, H, W, factor, k, _, stride, padding, dilation = shape
    return (batch, in_channel, H, W, factor, k, stride, padding, dilation)


if __name__ == "__main__":
    main("conv2d", "depthwise", depthwise_conv2d, shapes, args_of, trials_of=lambda t: [max(t // 10, 1), t])
