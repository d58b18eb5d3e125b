"""FusedConv2D, Conv2D, FusedDepthwiseConv2D, DepthwiseConv2dNative.

Reference kernels: tfjs-backend-cpu/src/kernels/FusedConv2D.ts:26-95,
Conv2D.ts:23-103, FusedDepthwiseConv2D.ts:25-61, DepthwiseConv2dNative.ts:23-102.
The geometry is computed on the host with computeConv2DInfo, as the reference's
WASM backend does before calling into C
(tfjs-backend-wasm/src/kernels/FusedConv2D.ts:79-147).
"""
from ctypes import byref

from .. import _cabi, conv_util
from ..backend import PendingConv, PendingDepthwise
from ..util import size_from_shape
from ..kernel_registry import KernelConfig
from .common import BACKEND, assert_not_complex, dev, per_channel_len, require_float32
from . import elementwise, movement


def _params(ci, activation, bias_len, prelu_len, alpha, depthwise=False):
    p = _cabi.Conv2DParams()
    p.batch, p.in_h, p.in_w, p.in_c = ci.batchSize, ci.inHeight, ci.inWidth, ci.inChannels
    p.out_h, p.out_w, p.out_c = ci.outHeight, ci.outWidth, ci.outChannels
    p.filter_h, p.filter_w = ci.filterHeight, ci.filterWidth
    p.stride_h, p.stride_w = ci.strideHeight, ci.strideWidth
    p.dilation_h, p.dilation_w = ci.dilationHeight, ci.dilationWidth
    p.pad_top, p.pad_left = int(ci.padInfo["top"]), int(ci.padInfo["left"])
    p.activation = _cabi.ACTIVATIONS[activation]
    p.bias_len, p.prelu_len = bias_len, prelu_len
    p.leakyrelu_alpha = 0.2 if alpha is None else float(alpha)
    return p


def _conv_impl(backend, x, filt, bias, prelu, attrs, activation, depthwise):
    name = "fused depthwiseConv2d" if depthwise else "fused conv2d"
    assert_not_complex([x, filt], name)
    require_float32(x, name)
    require_float32(filt, name)
    data_format = attrs.get("dataFormat") or "NHWC"
    if data_format not in ("NHWC", "NCHW"):
        raise ValueError("Unknown dataFormat %s" % data_format)
    nchw = data_format == "NCHW"
    if nchw and depthwise:
        raise ValueError("%s: the CUDA backend supports NHWC only, got NCHW" % name)
    strides = attrs.get("strides", 1)
    dilations = attrs.get("dilations")
    if dilations is None:
        dilations = [1, 1]
    pad = attrs.get("pad", "valid")
    rounding = attrs.get("dimRoundingMode")
    alpha = attrs.get("leakyreluAlpha")
    x_nhwc = x
    tmp = []
    if nchw:
        x_nhwc = movement.transpose_impl(backend, x, [0, 2, 3, 1])
        tmp.append(x_nhwc)
        if isinstance(pad, (list, tuple)):
            pad = [pad[0], pad[2], pad[3], pad[1]]
    ci = conv_util.compute_conv2d_info(x_nhwc.shape, filt.shape, strides, dilations, pad,
                                       rounding, depthwise)
    if not depthwise and filt.shape[2] != ci.inChannels:
        raise ValueError("Error in conv2d: depth of input (%d) must match input depth for "
                         "filter %d." % (ci.inChannels, filt.shape[2]))
    out_c = ci.outChannels
    bias_len = per_channel_len(bias, out_c)
    prelu_len = per_channel_len(prelu, out_c) if activation == "prelu" else 0
    if nchw:
        # NCHW bias / PReLU weights of shape [C], [C,1,1] broadcast per channel
        # (FusedConv2D.ts:55-61, :76-86).
        def nchw_len(t):
            if t is None:
                return 0
            n = 1
            for s in t.shape:
                n *= s
            if n == 1:
                return 1
            squeezed = [s for s in t.shape if s != 1]
            return out_c if squeezed == [out_c] and (len(t.shape) == 1 or
                                                      t.shape[-1] == 1) else None
        bias_len = nchw_len(bias)
        prelu_len = nchw_len(prelu) if activation == "prelu" else 0
    fuse_bias = bias_len is not None
    fuse_act = activation != "prelu" or prelu_len is not None
    if not fuse_bias:
        fuse_act = False  # the activation must come after the unfused add
    if (not fuse_bias or not fuse_act) and nchw:
        raise ValueError("%s: this bias / PReLU weight shape is not supported with NCHW "
                         "in the CUDA backend" % name)
    p = _params(ci, activation if fuse_act else "linear", bias_len if fuse_bias else 0,
                (prelu_len or 0) if fuse_act else 0, alpha, depthwise)
    if (backend.lazy_fusion and not depthwise and not nchw and fuse_bias and
            activation == "linear" and size_from_shape(ci.outShape) > 0):
        # Deferred: a following Add and / or Relu folds into this launch's epilogue.
        desc = {"name": "FusedConv2D",
                "inputShapes": dict([("x", list(x.shape)), ("filter", list(filt.shape))] +
                                    ([("bias", list(bias.shape))] if bias is not None else [])),
                "outputShapes": [list(ci.outShape)], "attrs": {}}
        return backend.defer(ci.outShape, "float32", PendingConv(
            p, x.dataId, filt.dataId, bias.dataId if bias is not None else None, None, [desc]))
    if (backend.lazy_fusion and depthwise and fuse_bias and
            activation in ("linear", "relu", "relu6") and size_from_shape(ci.outShape) > 0):
        # Deferred: the bias Add and the Relu / Relu6 that tfjs-layers issues after a
        # depthwise convolution fold into this launch, and a 1x1 convolution that consumes
        # the result (the projection of an inverted-residual block) absorbs the whole
        # depthwise convolution into its own launch.
        desc = {"name": "FusedDepthwiseConv2D" if bias is not None else "DepthwiseConv2dNative",
                "inputShapes": dict([("x", list(x.shape)), ("filter", list(filt.shape))] +
                                    ([("bias", list(bias.shape))] if bias is not None else [])),
                "outputShapes": [list(ci.outShape)], "attrs": {}}
        return backend.defer(ci.outShape, "float32", PendingDepthwise(
            p, x.dataId, filt.dataId, bias.dataId if bias is not None else None, [desc],
            activation))
    out = backend.make_output(ci.outShape, "float32")
    fn = (backend.lib.tfjs_cuda_fused_depthwise_conv2d if depthwise
          else backend.lib.tfjs_cuda_fused_conv2d)
    try:
        backend.check(fn(backend.ctx, byref(p), dev(backend, x_nhwc), dev(backend, filt),
                         dev(backend, bias) if fuse_bias and bias is not None else 0,
                         dev(backend, prelu) if fuse_act and activation == "prelu" else 0,
                         dev(backend, out)))
    except Exception:
        backend.disposeData(out.dataId)
        for t in tmp:
            backend.disposeData(t.dataId)
        raise
    for t in tmp:
        backend.disposeData(t.dataId)
    # Unfused tail, in the reference's order: Add, then the activation.
    if not fuse_bias:
        added = elementwise.binary_impl(backend, "Add", out, bias)
        backend.disposeData(out.dataId)
        out = added
    if not fuse_act:
        act = elementwise.apply_activation(backend, out, activation, prelu, alpha)
        backend.disposeData(out.dataId)
        out = act
    if nchw:
        back = movement.transpose_impl(backend, out, [0, 3, 1, 2])
        backend.disposeData(out.dataId)
        out = back
    return out


def fused_conv2d(args):
    i, a, b = args["inputs"], args["attrs"], args["backend"]
    return _conv_impl(b, i["x"], i["filter"], i.get("bias"),
                      i.get("preluActivationWeights"), a, a.get("activation") or "linear",
                      False)


def conv2d(args):
    i, a, b = args["inputs"], args["attrs"], args["backend"]
    return _conv_impl(b, i["x"], i["filter"], None, None, a, "linear", False)


def fused_depthwise_conv2d(args):
    i, a, b = args["inputs"], args["attrs"], args["backend"]
    return _conv_impl(b, i["x"], i["filter"], i.get("bias"),
                      i.get("preluActivationWeights"), a, a.get("activation") or "linear",
                      True)


def depthwise_conv2d_native(args):
    i, a, b = args["inputs"], args["attrs"], args["backend"]
    return _conv_impl(b, i["x"], i["filter"], None, None, a, "linear", True)


CONFIGS = [
    KernelConfig("FusedConv2D", BACKEND, fused_conv2d),
    KernelConfig("Conv2D", BACKEND, conv2d),
    KernelConfig("FusedDepthwiseConv2D", BACKEND, fused_depthwise_conv2d),
    KernelConfig("DepthwiseConv2dNative", BACKEND, depthwise_conv2d_native),
]
