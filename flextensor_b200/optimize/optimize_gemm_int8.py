"""int8 GEMM driver (the reference only has an AutoTVM tutorial for it,
flextensor/test/test_tvm/legacy/gemm_int8.py; same loop as optimize_gemm)."""
from ..configs.gemm_config import b200_gemm_int8_shapes
from ..task import gemm_int8
from .driver import main

shapes = list(b200_gemm_int8_shapes)

if __name__ == "__main__":
    main("gemm", "gemm_int8", gemm_int8, shapes, lambda shape: tuple(shape))
