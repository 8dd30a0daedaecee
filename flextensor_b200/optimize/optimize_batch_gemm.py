"""Batched GEMM bf16 driver (no counterpart script in the reference; same loop as optimize_gemm)."""
from ..configs.gemm_config import b200_batch_gemm_shapes
from ..task import batch_gemm
from .driver import main

shapes = list(b200_batch_gemm_shapes)

if __name__ == "__main__":
    main("gemm", "batch_gemm", batch_gemm, shapes, lambda shape: tuple(shape))
