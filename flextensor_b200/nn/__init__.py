from .ops import (zero_pad2d, zero_pad1d, gemm, batch_gemm, gemm_int8, conv2d_nchw, depthwise_conv2d_nchw, conv1d,
                  gemm_conv2d_nchw, conv2d_1x1_packed, relu, zero_pad3d, conv3d_ncdhw, conv2d_nhwc)
