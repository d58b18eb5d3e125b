"""tfjs_b200: a B200 (sm_100a) backend for the TensorFlow.js kernel contract.

Importing the package registers the 'cuda' backend and its kernels, the way
importing `@tensorflow/tfjs-backend-cpu` registers 'cpu'
(tfjs-backend-cpu/src/base.ts:31).  Priority 3 outranks webgl's 2
(tfjs-backend-webgl/src/base.ts:25).
"""
import os

from . import register_all_kernels  # noqa: F401  (side effect: registerKernel)
from .backend import CudaBackend, CudaError, TensorInfo  # noqa: F401
from .engine import ENGINE, Engine, Tensor  # noqa: F401


def _factory():
    return CudaBackend(int(os.environ.get("TFJS_CUDA_DEVICE_ORDINAL",
                                          os.environ.get("LOCAL_RANK", "0"))))


ENGINE.register_backend("cuda", _factory, 3)
