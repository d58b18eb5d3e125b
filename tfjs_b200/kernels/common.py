"""Helpers shared by the kernel funcs."""
from ctypes import byref

from .. import _cabi
from ..backend import TensorInfo
from ..util import size_from_shape

BACKEND = "cuda"


def dev(backend, info):
    """Device buffer id of a TensorInfo (0 when the optional input is absent)."""
    return backend.device_id(info.dataId) if info is not None else 0


def per_channel_len(info, channels):
    """Length to fuse a bias / PReLU weight tensor with: 1 for a scalar, `channels`
    for a tensor that broadcasts along the last axis, else None."""
    if info is None:
        return 0
    n = size_from_shape(info.shape)
    if n == 1:
        return 1
    if n == channels and len(info.shape) >= 1 and info.shape[-1] == channels:
        return channels
    return None


def view(backend, info, shape, dtype=None):
    """Zero-copy view: same dataId, one more reference (Reshape.ts:40-52)."""
    backend.incRef(info.dataId)
    return TensorInfo(info.dataId, shape, dtype or info.dtype)


def assert_not_complex(infos, name):
    """tfjs-backend-cpu/src/cpu_util.ts:20-34."""
    for t in (infos if isinstance(infos, (list, tuple)) else [infos]):
        if t is not None and t.dtype == "complex64":
            raise ValueError("%s does not support complex64 tensors in the CUDA backend." % name)


def require_float32(info, what):
    if info.dtype != "float32":
        raise ValueError("%s: the CUDA backend computes this kernel in float32, got %s" %
                         (what, info.dtype))
