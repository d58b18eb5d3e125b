"""Registers every kernel of the 'cuda' backend, like
tfjs-backend-cpu/src/register_all_kernels.ts does for 'cpu'."""
from .kernel_registry import register_kernel
from .kernels import conv, elementwise, matmul, movement, pool, reduce

ALL_CONFIGS = (conv.CONFIGS + matmul.CONFIGS + pool.CONFIGS + list(elementwise.CONFIGS) +
               reduce.CONFIGS + movement.CONFIGS)

for _cfg in ALL_CONFIGS:
    register_kernel(_cfg)
