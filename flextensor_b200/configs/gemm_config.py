"""GEMM shape tables (reference: flextensor/configs/gemm_config.py:11-31).

``gemm_shapes`` holds every (N, K, M) = (2^i, 2^k, 2^j) for i, j, k in 5..12, in the
reference's order (i outermost, then j, then k) so that list indices agree; it contains
the 1024^3 task of the README.  ``test_gemm_shapes`` are (batch, height, width, length)
batched cases.  ``b200_*`` are the extra shapes this backend is measured on.
"""
gemm_shapes = [[2 ** i, 2 ** k, 2 ** j] for i in range(5, 13) for j in range(5, 13) for k in range(5, 13)]

old_gemm_shapes = [(2 ** e,) * 3 for e in range(5, 12)]

test_gemm_shapes = [
    (1, 1024, 1024, 1024),
    (2, 512, 512, 512),
    (3, 1024, 32, 1024),
    (16, 4096, 128, 1024),
    (32, 28, 1024, 28),
]

# (batch, N, K, M): bf16 batched GEMM measured sharded over 1/2/4/8 GPUs
b200_batch_gemm_shapes = [(64, 2048, 2048, 2048), (8, 1024, 1024, 1024), (4, 256, 512, 384)]
# (N, K, M): int8 GEMM with int32 accumulation
b200_gemm_int8_shapes = [(8192, 8192, 8192), (4096, 4096, 4096), (1024, 1024, 1024), (256, 512, 384)]
