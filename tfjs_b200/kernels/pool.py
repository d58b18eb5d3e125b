"""MaxPool and AvgPool (tfjs-backend-cpu/src/kernels/MaxPool.ts:24-55,
AvgPool.ts:24-55, utils/pool_utils.ts:20-87)."""
from ctypes import byref

from .. import _cabi, conv_util
from ..kernel_registry import KernelConfig
from .common import BACKEND, assert_not_complex, dev, require_float32, view


def _pool(args, is_max):
    i, a, backend = args["inputs"], args["attrs"], args["backend"]
    x = i["x"]
    name = "maxPool" if is_max else "avgPool"
    assert_not_complex(x, name)
    require_float32(x, name)
    strides = a.get("strides", 1)
    dilations = 1
    if not conv_util.either_strides_or_dilations_are_one(strides, dilations):
        raise ValueError("Error in %s: Either strides or dilations must be 1." % name)
    ci = conv_util.compute_pool2d_info(x.shape, a["filterSize"], strides, dilations,
                                       a.get("pad", "valid"), a.get("dimRoundingMode"))
    if ci.filterWidth == 1 and ci.filterHeight == 1 and list(ci.inShape) == list(ci.outShape):
        return view(backend, x, x.shape)  # identity (MaxPool.ts:44-46)
    p = _cabi.Conv2DParams()
    p.batch, p.in_h, p.in_w, p.in_c = ci.batchSize, ci.inHeight, ci.inWidth, ci.inChannels
    p.out_h, p.out_w, p.out_c = ci.outHeight, ci.outWidth, ci.inChannels
    p.filter_h, p.filter_w = ci.effectiveFilterHeight, ci.effectiveFilterWidth
    p.stride_h, p.stride_w = ci.strideHeight, ci.strideWidth
    p.dilation_h, p.dilation_w = ci.dilationHeight, ci.dilationWidth
    p.pad_top, p.pad_left = int(ci.padInfo["top"]), int(ci.padInfo["left"])
    out = backend.make_output(ci.outShape, "float32")
    try:
        backend.check(backend.lib.tfjs_cuda_pool2d(backend.ctx, byref(p), int(is_max),
                                                   dev(backend, x), dev(backend, out)))
    except Exception:
        backend.disposeData(out.dataId)
        raise
    return out


CONFIGS = [
    KernelConfig("MaxPool", BACKEND, lambda args: _pool(args, True)),
    KernelConfig("AvgPool", BACKEND, lambda args: _pool(args, False)),
]
