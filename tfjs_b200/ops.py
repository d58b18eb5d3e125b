"""Op front ends: argument validation, rank lifting and attribute packing, then
ENGINE.run_kernel under the tfjs kernel names.

These mirror the tfjs-core ops that call the hot-path kernels (for a Node build
tfjs-core's own ops play this role): fused/conv2d.ts:96-330, fused/mat_mul.ts,
fused/depthwise_conv2d.ts, conv2d.ts, depthwise_conv2d.ts, mat_mul.ts:45-56,
max_pool.ts, avg_pool.ts, softmax.ts, mean.ts, gather.ts, ...
"""
import numpy as np

from . import conv_util
from .engine import ENGINE, Tensor
from .util import size_from_shape


def tensor(values, shape=None, dtype=None):
    return ENGINE.make_tensor(values, shape, dtype)


def _t(x, dtype=None):
    if isinstance(x, Tensor):
        return x, False
    return ENGINE.make_tensor(x, None, dtype), True


def _run(name, inputs, attrs=None):
    return ENGINE.run_kernel(name, inputs, attrs or {})


def _reshape_view(x, shape):
    return _run("Reshape", {"x": x}, {"shape": list(shape)})


def reshape(x, shape):
    return _reshape_view(x, shape)


# ------------------------------------------------------------- convolution --
def _check_conv_args(name, x4, f, strides, dilations, pad, dim_rounding, data_format):
    if x4.rank != 4:
        raise ValueError("Error in %s: input must be rank 4, but got rank %d." % (name, x4.rank))
    if f.rank != 4:
        raise ValueError("Error in %s: filter must be rank 4, but got rank %d." % (name, f.rank))
    conv_util.check_pad_on_dim_rounding_mode(name, pad, dim_rounding)
    if not conv_util.either_strides_or_dilations_are_one(strides, dilations):
        raise ValueError("Error in %s: Either strides or dilations must be 1. Got strides %s "
                         "and dilations '%s'" % (name, strides, dilations))
    for v in conv_util.parse_tuple_param(strides) + conv_util.parse_tuple_param(dilations):
        if v <= 0:
            raise ValueError("Error in %s: Strides and dilations should be greater than 0." % name)
    for t in (x4, f):
        if t.dtype != "float32":
            raise ValueError("Argument passed to '%s' must be float32 tensor, but got %s "
                             "tensor" % (name, t.dtype))


def fused_conv2d(x, filter, strides, pad, dataFormat="NHWC", dilations=(1, 1),
                 dimRoundingMode=None, bias=None, activation="linear",
                 preluActivationWeights=None, leakyreluAlpha=None):
    """tfjs-core/src/ops/fused/conv2d.ts:96-330."""
    x3 = x.rank == 3
    x4 = _reshape_view(x, [1] + x.shape) if x3 else x
    try:
        _check_conv_args("fused conv2d", x4, filter, strides, dilations, pad, dimRoundingMode,
                         dataFormat)
        in_depth = x4.shape[3] if dataFormat == "NHWC" else x4.shape[1]
        if in_depth != filter.shape[2]:
            raise ValueError("Error in conv2d: depth of input (%d) must match input depth for "
                             "filter %d." % (in_depth, filter.shape[2]))
        inputs = {"x": x4, "filter": filter, "bias": bias,
                  "preluActivationWeights": preluActivationWeights}
        attrs = {"strides": strides, "pad": pad, "dataFormat": dataFormat,
                 "dilations": list(dilations) if not isinstance(dilations, int) else dilations,
                 "dimRoundingMode": dimRoundingMode, "activation": activation,
                 "leakyreluAlpha": leakyreluAlpha}
        out = _run("FusedConv2D", inputs, attrs)
    finally:
        if x3:
            x4.dispose()
    if x3:
        r = _reshape_view(out, out.shape[1:])
        out.dispose()
        return r
    return out


def conv2d(x, filter, strides, pad, dataFormat="NHWC", dilations=(1, 1),
           dimRoundingMode=None):
    """tfjs-core/src/ops/conv2d.ts."""
    x3 = x.rank == 3
    x4 = _reshape_view(x, [1] + x.shape) if x3 else x
    try:
        _check_conv_args("conv2d", x4, filter, strides, dilations, pad, dimRoundingMode,
                         dataFormat)
        out = _run("Conv2D", {"x": x4, "filter": filter},
                   {"strides": strides, "pad": pad, "dataFormat": dataFormat,
                    "dilations": dilations, "dimRoundingMode": dimRoundingMode})
    finally:
        if x3:
            x4.dispose()
    if x3:
        r = _reshape_view(out, out.shape[1:])
        out.dispose()
        return r
    return out


def _depthwise(kernel, name, x, filter, strides, pad, dataFormat, dilations,
               dimRoundingMode, extra_inputs=None, extra_attrs=None):
    x3 = x.rank == 3
    x4 = _reshape_view(x, [1] + x.shape) if x3 else x
    try:
        if dilations is None:
            dilations = [1, 1]
        _check_conv_args(name, x4, filter, strides, dilations, pad, dimRoundingMode, dataFormat)
        if x4.shape[3] != filter.shape[2]:
            raise ValueError("Error in %s: number of input channels (%d) must match the "
                             "inChannels dimension in filter %d." %
                             (name, x4.shape[3], filter.shape[2]))
        inputs = {"x": x4, "filter": filter}
        inputs.update(extra_inputs or {})
        attrs = {"strides": strides, "pad": pad, "dataFormat": dataFormat,
                 "dilations": dilations, "dimRoundingMode": dimRoundingMode}
        attrs.update(extra_attrs or {})
        out = _run(kernel, inputs, attrs)
    finally:
        if x3:
            x4.dispose()
    if x3:
        r = _reshape_view(out, out.shape[1:])
        out.dispose()
        return r
    return out


def depthwise_conv2d(x, filter, strides, pad, dataFormat="NHWC", dilations=(1, 1),
                     dimRoundingMode=None):
    """tfjs-core/src/ops/depthwise_conv2d.ts."""
    return _depthwise("DepthwiseConv2dNative", "depthwiseConv2d", x, filter, strides, pad,
                      dataFormat, dilations, dimRoundingMode)


def fused_depthwise_conv2d(x, filter, strides, pad, dataFormat="NHWC", dilations=(1, 1),
                           dimRoundingMode=None, bias=None, activation="linear",
                           preluActivationWeights=None, leakyreluAlpha=None):
    """tfjs-core/src/ops/fused/depthwise_conv2d.ts."""
    return _depthwise("FusedDepthwiseConv2D", "fused depthwiseConv2d", x, filter, strides, pad,
                      dataFormat, dilations, dimRoundingMode,
                      {"bias": bias, "preluActivationWeights": preluActivationWeights},
                      {"activation": activation, "leakyreluAlpha": leakyreluAlpha})


# ------------------------------------------------------------------ matmul --
def mat_mul(a, b, transposeA=False, transposeB=False):
    """tfjs-core/src/ops/mat_mul.ts:45-56: tensors go to the kernel unchanged."""
    return _run("BatchMatMul", {"a": a, "b": b},
                {"transposeA": transposeA, "transposeB": transposeB})


def mat_mul_heads(a, b, layout, heads, transposeA=False, transposeB=False, bias=None,
                  activation="linear", preluActivationWeights=None, leakyreluAlpha=0.2):
    """matMul whose result is stored with attention heads split ("split": [B*S, H*D] product
    written as [B, H, S, D]) or merged ("merge": [B, H, S, D] product written as
    [B, S, H, D]); heads = [B, S, H, D].  A kernel of the 'cuda' backend with no counterpart
    among the reference's ops (the graph executor substitutes it for matMul + reshape +
    transpose); raises CudaError(UNSUPPORTED) for shapes it does not take."""
    return _run("_MatMulHeads", {"a": a, "b": b, "bias": bias,
                                 "preluActivationWeights": preluActivationWeights},
                {"transposeA": transposeA, "transposeB": transposeB, "activation": activation,
                 "leakyreluAlpha": leakyreluAlpha, "layout": layout, "heads": list(heads)})


def fused_mat_mul(a, b, transposeA=False, transposeB=False, bias=None, activation="linear",
                  preluActivationWeights=None, leakyreluAlpha=0.2, geluParams=None):
    """tfjs-core/src/ops/fused/mat_mul.ts: operands are reshaped to rank 3 first
    (:117-122) and the result is reshaped back.  activation "gelu_erf" with geluParams =
    [scale, half, one, divide] exists on the 'cuda' backend only: (h * half) * (erf(h * scale)
    + one) as the epilogue (the graph executor substitutes it for the five nodes of an erf
    GELU after a dense layer)."""
    inner_a = a.shape[a.rank - 2] if transposeA else a.shape[a.rank - 1]
    inner_b = b.shape[b.rank - 1] if transposeB else b.shape[b.rank - 2]
    outer_a = a.shape[a.rank - 1] if transposeA else a.shape[a.rank - 2]
    outer_b = b.shape[b.rank - 2] if transposeB else b.shape[b.rank - 1]
    if inner_a != inner_b:
        raise ValueError(
            "Error in fused matMul: inner shapes (%d) and (%d) of Tensors with shapes %s and "
            "%s and transposeA=%s and transposeB=%s must match." %
            (inner_a, inner_b, a.shape, b.shape, transposeA, transposeB))
    from .util import assert_and_get_broadcast_shape
    out_dims = assert_and_get_broadcast_shape(a.shape[:-2], b.shape[:-2])
    out_shape = out_dims + [outer_a, outer_b]
    batch_a, batch_b = size_from_shape(a.shape[:-2]), size_from_shape(b.shape[:-2])
    a3 = _reshape_view(a, [batch_a] + a.shape[-2:])
    b3 = _reshape_view(b, [batch_b] + b.shape[-2:])
    try:
        if bias is not None:
            assert_and_get_broadcast_shape(out_shape, bias.shape)
        out = _run("_FusedMatMul",
                   {"a": a3, "b": b3, "bias": bias,
                    "preluActivationWeights": preluActivationWeights},
                   {"transposeA": transposeA, "transposeB": transposeB,
                    "activation": activation, "leakyreluAlpha": leakyreluAlpha,
                    "geluParams": geluParams})
    finally:
        a3.dispose()
        b3.dispose()
    r = _reshape_view(out, out_shape)
    out.dispose()
    return r


# ----------------------------------------------------------------- pooling --
def _pool(kernel, name, x, filterSize, strides, pad, dimRoundingMode):
    x3 = x.rank == 3
    x4 = _reshape_view(x, [1] + x.shape) if x3 else x
    try:
        if x4.rank != 4:
            raise ValueError("Error in %s: x must be rank 4 but got rank %d." % (name, x4.rank))
        conv_util.check_pad_on_dim_rounding_mode(name, pad, dimRoundingMode)
        out = _run(kernel, {"x": x4}, {"filterSize": filterSize, "strides": strides, "pad": pad,
                                       "dimRoundingMode": dimRoundingMode})
    finally:
        if x3:
            x4.dispose()
    if x3:
        r = _reshape_view(out, out.shape[1:])
        out.dispose()
        return r
    return out


def max_pool(x, filterSize, strides, pad, dimRoundingMode=None):
    return _pool("MaxPool", "maxPool", x, filterSize, strides, pad, dimRoundingMode)


def avg_pool(x, filterSize, strides, pad, dimRoundingMode=None):
    return _pool("AvgPool", "avgPool", x, filterSize, strides, pad, dimRoundingMode)


# ------------------------------------------------------------- elementwise --
def _binary(name):
    def f(a, b):
        return _run(name, {"a": a, "b": b})
    return f


add = _binary("Add")
sub = _binary("Sub")
mul = _binary("Multiply")
div = _binary("RealDiv")
maximum = _binary("Maximum")
minimum = _binary("Minimum")
pow = _binary("Pow")
squared_difference = _binary("SquaredDifference")


def prelu(x, alpha):
    return _run("Prelu", {"x": x, "alpha": alpha})


def _unary(name):
    def f(x):
        return _run(name, {"x": x})
    return f


relu = _unary("Relu")
relu6 = _unary("Relu6")
elu = _unary("Elu")
sigmoid = _unary("Sigmoid")
exp = _unary("Exp")
sqrt = _unary("Sqrt")
rsqrt = _unary("Rsqrt")
square = _unary("Square")
tanh = _unary("Tanh")
neg = _unary("Neg")
erf = _unary("Erf")
abs = _unary("Abs")
log = _unary("Log")


def leaky_relu(x, alpha=0.2):
    return _run("LeakyRelu", {"x": x}, {"alpha": alpha})


def clip_by_value(x, lo, hi):
    if lo > hi:
        raise ValueError("Error in clip: min (%s) must be less than or equal to max (%s)." %
                         (lo, hi))
    return _run("ClipByValue", {"x": x}, {"clipValueMin": lo, "clipValueMax": hi})


def batch_norm(x, mean, variance, offset=None, scale=None, varianceEpsilon=None):
    return _run("FusedBatchNorm", {"x": x, "mean": mean, "variance": variance,
                                   "offset": offset, "scale": scale},
                {"varianceEpsilon": varianceEpsilon})


def cast(x, dtype):
    return _run("Cast", {"x": x}, {"dtype": dtype})


# -------------------------------------------------------------- reductions --
def softmax(logits, dim=-1):
    return _run("Softmax", {"logits": logits}, {"dim": dim})


def softmax_scaled_masked(logits, scale=None, mask=None):
    """softmax(logits * scale + mask) over the last axis as one kernel of the 'cuda' backend
    (the graph executor substitutes it for Mul + AddV2 + Softmax); the mask must broadcast
    over whole rows."""
    return _run("_SoftmaxScaledMasked", {"logits": logits, "mask": mask}, {"scale": scale})


def fused_attention(q, k, v, scale=None, mask=None):
    """softmax(q k^T * scale + mask) v for q, k, v of shape [B, H, S, D], returned as
    [B, S, H, D]: one kernel of the 'cuda' backend with no counterpart among the
    reference's ops (the graph executor substitutes it for batchMatMul + mul + add + softmax
    + batchMatMul + transpose); raises CudaError(UNSUPPORTED) for shapes it does not take."""
    return _run("_FusedAttention", {"q": q, "k": k, "v": v, "mask": mask}, {"scale": scale})


def fused_layer_norm(x, gamma, beta, epsilon, residual=None):
    """Layer normalisation over the last axis in the decomposed form of a converted graph,
    as one kernel of the 'cuda' backend (no counterpart among the reference's ops; the
    graph executor substitutes it for the matched subgraph)."""
    return _run("_FusedLayerNorm", {"x": x, "gamma": gamma, "beta": beta, "residual": residual},
                {"epsilon": float(epsilon)})


def sum(x, axis=None, keepDims=False):
    return _run("Sum", {"x": x}, {"axis": axis, "keepDims": keepDims})


def mean(x, axis=None, keepDims=False):
    return _run("Mean", {"x": x}, {"axis": axis, "keepDims": keepDims})


def max(x, axis=None, keepDims=False):
    return _run("Max", {"x": x}, {"reductionIndices": axis, "keepDims": keepDims})


def arg_max(x, axis=0):
    return _run("ArgMax", {"x": x}, {"axis": axis})


# ---------------------------------------------------------------- movement --
def transpose(x, perm=None):
    if perm is None:
        perm = list(range(x.rank))[::-1]
    return _run("Transpose", {"x": x}, {"perm": list(perm)})


def expand_dims(x, axis=0):
    return _run("ExpandDims", {"input": x}, {"dim": axis})


def identity(x):
    return _run("Identity", {"x": x})


def gather(x, indices, axis=0, batchDims=0):
    return _run("GatherV2", {"x": x, "indices": indices}, {"axis": axis, "batchDims": batchDims})


def concat(tensors, axis=0):
    return ENGINE.run_kernel("Concat", {str(i): t for i, t in enumerate(tensors)},
                             {"axis": axis})


def stack(tensors, axis=0):
    return ENGINE.run_kernel("Pack", {str(i): t for i, t in enumerate(tensors)}, {"axis": axis})


def slice(x, begin, size=None):
    return _run("Slice", {"x": x}, {"begin": begin, "size": size})


def pad(x, paddings, constantValue=0):
    return _run("PadV2", {"x": x}, {"paddings": paddings, "constantValue": constantValue})


def tile(x, reps):
    return _run("Tile", {"x": x}, {"reps": list(reps)})
