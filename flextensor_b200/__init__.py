"""flextensor_b200: B200 (sm_100a) kernel backend behind FlexTensor's Python interface.

  nn.ops        compute definitions (gemm, batch_gemm, gemm_int8, conv2d_nchw, depthwise_conv2d_nchw)
  task          Task / register_task / TASK_TABLE and the registered shapes
  space         config space: kernel knobs (tile, cluster, stages, raster, split-K)
  scheduler     schedule / schedule_with_config (heuristic and Q-learning search)
  model         walkers (DQN) and performance model
  measure       candidate measurement, one per GPU
  runtime       KernelPlan, Module, build: the callable that replaces tvm.build's output
  backend       ctypes binding of the C ABI (include/ftb200.h); csrc/ holds the CUDA sources
  sharded       batch-sharded execution over several GPUs with an NCCL all-gather of the output
"""
__version__ = "0.1.0"
