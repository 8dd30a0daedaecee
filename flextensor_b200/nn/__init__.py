from .ops import (zero_pad2d, gemm, batch_gemm, gemm_int8, conv2d_nchw, depthwise_conv2d_nchw)
