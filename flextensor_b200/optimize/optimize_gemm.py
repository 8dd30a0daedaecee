"""GEMM fp32 driver (flextensor/optimize/optimize_gemm.py): ``python -m flextensor_b200.optimize.optimize_gemm``."""
from ..task import gemm
from .driver import main

shapes = [(256, 128, 128), (256, 256, 256), (1024, 1024, 1024)]

if __name__ == "__main__":
    main("gemm", "gemm", gemm, shapes, lambda shape: tuple(shape))
