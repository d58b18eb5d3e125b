"""TEST INFRASTRUCTURE ONLY -- numpy/ctypes front end of the CPU oracle.

A CPU restatement of the tfjs-backend-cpu kernels on the inference hot path.
Only tests, the smoke check and the CPU-baseline legs of the benchmark may
import this module; the CUDA product path never does.

Arithmetic lives in tfjs_cpu_oracle.c (double math, fp32 stores, reference
accumulation order).  Exact data movement (transpose, gather, concat, slice,
pad, tile) is numpy indexing.  Shape rules are restated here independently of
the product's host code so that the two cross-check each other.

Parity status: pinned by tests/test_oracle_golden.py against the reference's own
op-test vectors and quantization.py fixtures.
"""
import ctypes
import math
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libtfjs_cpu_oracle.so")
_lib = None

c_long_p = ctypes.POINTER(ctypes.c_long)


def build():
    """Compile the C restatement with the Makefile beside it."""
    subprocess.check_call(["make", "-s", "-C", _HERE])


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = ctypes.CDLL(_LIB_PATH)
        _lib.orc_max_threads.restype = ctypes.c_int
    return _lib


def set_threads(n):
    lib().orc_set_threads(int(n))


def max_threads():
    return int(lib().orc_max_threads())


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _ptr(a):
    return a.ctypes.data_as(ctypes.c_void_p)


# ---------------------------------------------------------------- shape rules
def _pair(v):
    if isinstance(v, (int, np.integer)):
        return int(v), int(v)
    v = list(v)
    if len(v) == 1:
        return int(v[0]), int(v[0])
    return int(v[0]), int(v[1])


def _js_round(v):
    r = math.floor(v)
    return r + 1 if v - r >= 0.5 else r


def _round(value, mode):
    """tfjs-core/src/ops/conv_util.ts:548-564."""
    if not mode:
        return math.trunc(value)
    if mode == "round":
        return _js_round(value)
    if mode == "ceil":
        return math.ceil(value)
    if mode == "floor":
        return math.floor(value)
    raise ValueError("Unknown roundingMode %s" % mode)


def conv2d_info(in_shape, filter_shape, strides, dilations, pad,
                rounding_mode=None, depthwise=False):
    """tfjs-core/src/ops/conv_util.ts:177-236 and :429-481 (NHWC only)."""
    batch, in_h, in_w, in_c = [int(v) for v in in_shape]
    f_h, f_w, _, f_c = [int(v) for v in filter_shape]
    s_h, s_w = _pair(strides)
    d_h, d_w = _pair(dilations)
    eff_h = f_h if d_h <= 1 else f_h + (f_h - 1) * (d_h - 1)
    eff_w = f_w if d_w <= 1 else f_w + (f_w - 1) * (d_w - 1)
    if isinstance(pad, (int, np.integer)):
        pad = int(pad)
        top = bottom = left = right = pad
        # conv_util.ts:350-365 uses the height's field size and stride for both
        # output dimensions.
        out_h = _round((in_h - eff_h + 2 * pad) / s_h + 1, rounding_mode)
        out_w = _round((in_w - eff_h + 2 * pad) / s_h + 1, rounding_mode)
    elif pad == "same":
        out_h = math.ceil(in_h / s_h)
        out_w = math.ceil(in_w / s_w)
        pad_h = max(0, (out_h - 1) * s_h + eff_h - in_h)
        pad_w = max(0, (out_w - 1) * s_w + eff_w - in_w)
        top = pad_h // 2
        bottom = pad_h - top
        left = pad_w // 2
        right = pad_w - left
    elif pad == "valid":
        top = bottom = left = right = 0
        out_h = math.ceil((in_h - eff_h + 1) / s_h)
        out_w = math.ceil((in_w - eff_w + 1) / s_w)
    else:
        top, bottom = int(pad[1][0]), int(pad[1][1])
        left, right = int(pad[2][0]), int(pad[2][1])
        out_h = _round((in_h - eff_h + top + bottom) / s_h + 1, rounding_mode)
        out_w = _round((in_w - eff_w + left + right) / s_w + 1, rounding_mode)
    out_c = f_c * in_c if depthwise else f_c
    return dict(batch=batch, in_h=in_h, in_w=in_w, in_c=in_c, out_h=out_h,
                out_w=out_w, out_c=out_c, f_h=f_h, f_w=f_w, s_h=s_h, s_w=s_w,
                d_h=d_h, d_w=d_w, eff_h=eff_h, eff_w=eff_w, top=top,
                bottom=bottom, left=left, right=right,
                out_shape=(batch, out_h, out_w, out_c))


def broadcast_shape(a, b):
    """tfjs-core/src/ops/broadcast_util.ts:65-100."""
    out = []
    n = max(len(a), len(b))
    for i in range(n):
        x = a[len(a) - 1 - i] if i < len(a) else 1
        y = b[len(b) - 1 - i] if i < len(b) else 1
        if x == 1:
            out.insert(0, y)
        elif y == 1:
            out.insert(0, x)
        elif x != y:
            raise ValueError("Operands could not be broadcast together with "
                             "shapes %s and %s." % (list(a), list(b)))
        else:
            out.insert(0, x)
    return tuple(out)


# ------------------------------------------------------------------- kernels
def conv2d(x, w, strides=1, pad="valid", dilations=1, rounding_mode=None):
    x, w = _f32(x), _f32(w)
    ci = conv2d_info(x.shape, w.shape, strides, dilations, pad, rounding_mode)
    y = np.empty(ci["out_shape"], np.float32)
    lib().orc_conv2d(_ptr(x), _ptr(w), _ptr(y), ci["batch"], ci["in_h"],
                     ci["in_w"], ci["in_c"], ci["out_h"], ci["out_w"],
                     ci["out_c"], ci["f_h"], ci["f_w"], ci["s_h"], ci["s_w"],
                     ci["d_h"], ci["d_w"], ci["top"], ci["left"])
    return y


def depthwise_conv2d(x, w, strides=1, pad="valid", dilations=1,
                     rounding_mode=None):
    x, w = _f32(x), _f32(w)
    ci = conv2d_info(x.shape, w.shape, strides, dilations, pad, rounding_mode,
                     depthwise=True)
    y = np.empty(ci["out_shape"], np.float32)
    lib().orc_depthwise_conv2d(_ptr(x), _ptr(w), _ptr(y), ci["batch"],
                               ci["in_h"], ci["in_w"], ci["in_c"],
                               int(w.shape[3]), ci["out_h"], ci["out_w"],
                               ci["f_h"], ci["f_w"], ci["s_h"], ci["s_w"],
                               ci["d_h"], ci["d_w"], ci["top"], ci["left"])
    return y


def batch_matmul(a, b, transpose_a=False, transpose_b=False):
    """BatchMatMul.ts:25-133: any rank >= 2, outer dims broadcast."""
    a, b = _f32(a), _f32(b)
    inner_a = a.shape[-2] if transpose_a else a.shape[-1]
    inner_b = b.shape[-1] if transpose_b else b.shape[-2]
    outer_a = a.shape[-1] if transpose_a else a.shape[-2]
    outer_b = b.shape[-2] if transpose_b else b.shape[-1]
    if inner_a != inner_b:
        raise ValueError("Error in matMul: inner shapes (%d) and (%d) must "
                         "match." % (inner_a, inner_b))
    batch_a = int(np.prod(a.shape[:-2], dtype=np.int64))
    batch_b = int(np.prod(b.shape[:-2], dtype=np.int64))
    out_outer = broadcast_shape(a.shape[:-2], b.shape[:-2])
    batch = max(batch_a, batch_b)
    out = np.zeros((batch, outer_a, outer_b), np.float32)
    if out.size and inner_a:
        lib().orc_batch_matmul(_ptr(a), _ptr(b), _ptr(out), batch_a, batch_b,
                               outer_a, outer_b, inner_a, int(transpose_a),
                               int(transpose_b))
    return out.reshape(tuple(out_outer) + (outer_a, outer_b))


_UNARY = dict(relu=0, relu6=1, elu=2, sigmoid=3, leakyrelu=4, exp=5, sqrt=6,
              rsqrt=7, square=8, tanh=9, neg=10, clip=11, erf=12, abs=13,
              log=14, linear=15, identity=15)
_BINARY = dict(add=0, sub=1, mul=2, div=3, maximum=4, minimum=5, pow=6,
               squared_difference=7, prelu=8)


def unary(op, x, p0=0.0, p1=0.0):
    x = _f32(x)
    y = np.empty_like(x)
    lib().orc_unary(_UNARY[op], _ptr(x), _ptr(y), ctypes.c_long(x.size),
                    ctypes.c_double(p0), ctypes.c_double(p1))
    return y


def binary(op, a, b):
    a, b = np.asarray(a), np.asarray(b)
    is_int = a.dtype == np.int32 and b.dtype == np.int32
    dt = np.int32 if is_int else np.float32
    a = np.ascontiguousarray(a, dt)
    b = np.ascontiguousarray(b, dt)
    out_shape = broadcast_shape(a.shape, b.shape)
    rank = max(len(out_shape), 1)
    pad = lambda s: (1,) * (rank - len(s)) + tuple(s)
    arr = lambda s: (ctypes.c_long * rank)(*pad(s))
    out = np.empty(out_shape, dt)
    fn = lib().orc_binary_i32 if is_int else lib().orc_binary_f32
    if out.size:
        fn(_BINARY[op], _ptr(a), arr(a.shape), _ptr(b), arr(b.shape),
           _ptr(out), arr(out_shape), rank)
    return out


def apply_activation(x, activation, prelu_weights=None, leakyrelu_alpha=None):
    """tfjs-backend-cpu/src/utils/fused_utils.ts:29-49."""
    if activation in (None, "linear"):
        return _f32(x)
    if activation == "prelu":
        return binary("prelu", x, prelu_weights)
    if activation == "leakyrelu":
        return unary("leakyrelu", x, float(leakyrelu_alpha))
    if activation in ("relu", "relu6", "elu", "sigmoid"):
        return unary(activation, x)
    raise ValueError("Activation %s has not been implemented" % activation)


def fused_conv2d(x, w, strides=1, pad="valid", dilations=1, rounding_mode=None,
                 bias=None, activation="linear", prelu_weights=None,
                 leakyrelu_alpha=None):
    """FusedConv2D.ts:26-95: conv2D, then Add, then the activation, each an
    fp32-rounded pass."""
    y = conv2d(x, w, strides, pad, dilations, rounding_mode)
    if bias is not None:
        y = binary("add", y, bias)
    return apply_activation(y, activation, prelu_weights, leakyrelu_alpha)


def fused_depthwise_conv2d(x, w, strides=1, pad="valid", dilations=1,
                           rounding_mode=None, bias=None, activation="linear",
                           prelu_weights=None, leakyrelu_alpha=None):
    """FusedDepthwiseConv2D.ts:25-61."""
    y = depthwise_conv2d(x, w, strides, pad, dilations, rounding_mode)
    if bias is not None:
        y = binary("add", y, bias)
    return apply_activation(y, activation, prelu_weights, leakyrelu_alpha)


def fused_matmul(a, b, transpose_a=False, transpose_b=False, bias=None,
                 activation="linear", prelu_weights=None, leakyrelu_alpha=None):
    """_FusedMatMul.ts:26-62."""
    y = batch_matmul(a, b, transpose_a, transpose_b)
    if bias is not None:
        y = binary("add", y, bias)
    return apply_activation(y, activation, prelu_weights, leakyrelu_alpha)


def pool2d(x, kind, filter_size, strides, pad, rounding_mode=None,
           dilations=1):
    """MaxPool.ts:24-55 / AvgPool.ts:24-55 over utils/pool_utils.ts:20-87."""
    x = _f32(x)
    f_h, f_w = _pair(filter_size)
    ci = conv2d_info(x.shape, (f_h, f_w, x.shape[3], x.shape[3]), strides,
                     dilations, pad, rounding_mode)
    if (ci["f_h"] == 1 and ci["f_w"] == 1 and
            tuple(ci["out_shape"]) == tuple(x.shape)):
        return x.copy()
    y = np.empty(ci["out_shape"], np.float32)
    lib().orc_pool2d(_ptr(x), _ptr(y), int(kind == "max"), ci["batch"],
                     ci["in_h"], ci["in_w"], ci["in_c"], ci["out_h"],
                     ci["out_w"], ci["eff_h"], ci["eff_w"], ci["s_h"],
                     ci["s_w"], ci["d_h"], ci["d_w"], ci["top"], ci["left"])
    return y


def _norm_axes(axis, rank):
    if axis is None:
        return list(range(rank))
    if isinstance(axis, (int, np.integer)):
        axis = [int(axis)]
    return [int(a) % rank if rank else 0 for a in axis]


def _rows_view(x, axes):
    """Move the reduced axes innermost (axis_util.ts:86-110) and flatten."""
    rank = x.ndim
    axes = sorted(axes)
    keep = [d for d in range(rank) if d not in axes]
    xt = np.ascontiguousarray(np.transpose(x, keep + axes))
    out_shape = tuple(x.shape[d] for d in keep)
    reduce_size = int(np.prod([x.shape[d] for d in axes], dtype=np.int64))
    return xt, out_shape, reduce_size


def _keep(shape, out_shape, axes, rank, keep_dims):
    if not keep_dims:
        return out_shape
    return tuple(1 if d in axes else shape[d] for d in range(rank))


def reduce(op, x, axis=None, keep_dims=False):
    """Sum.ts:28-90, Mean.ts:25-53, Max.ts:28-72."""
    x = _f32(x)
    axes = _norm_axes(axis, x.ndim)
    xt, out_shape, rs = _rows_view(x, axes)
    rows = int(np.prod(out_shape, dtype=np.int64))
    y = np.empty(rows, np.float32)
    fn = dict(sum=lib().orc_sum_rows, mean=lib().orc_mean_rows,
              max=lib().orc_max_rows)[op]
    fn(_ptr(xt), _ptr(y), ctypes.c_long(rows), ctypes.c_long(rs))
    return y.reshape(_keep(x.shape, out_shape, axes, x.ndim, keep_dims))


def argmax(x, axis=0):
    """ArgMax.ts:24-71."""
    x = _f32(x)
    axes = _norm_axes(axis, x.ndim)[:1]
    xt, out_shape, rs = _rows_view(x, axes)
    rows = int(np.prod(out_shape, dtype=np.int64))
    y = np.empty(rows, np.int32)
    lib().orc_argmax_rows(_ptr(xt), _ptr(y), ctypes.c_long(rows),
                          ctypes.c_long(rs))
    return y.reshape(out_shape)


def softmax(x, dim=-1):
    """Softmax.ts:29-77 (last dimension only)."""
    x = _f32(x)
    if dim not in (-1, x.ndim - 1):
        raise ValueError("Softmax along a non-last dimension is not yet "
                         "supported.")
    y = np.empty_like(x)
    cols = x.shape[-1]
    lib().orc_softmax_rows(_ptr(x), _ptr(y), ctypes.c_long(x.size // cols),
                           ctypes.c_long(cols))
    return y


def batch_norm(x, mean, variance, offset=None, scale=None, eps=None):
    """BatchNorm.ts:23-90."""
    x, mean, variance = _f32(x), _f32(mean), _f32(variance)
    eps = 0.001 if eps is None else eps
    off = _f32(offset) if offset is not None else None
    sc = _f32(scale) if scale is not None else None
    y = np.empty_like(x)
    lib().orc_batchnorm(_ptr(x), _ptr(mean), ctypes.c_long(mean.size),
                        _ptr(variance), ctypes.c_long(variance.size),
                        _ptr(sc) if sc is not None else None,
                        ctypes.c_long(sc.size if sc is not None else 1),
                        _ptr(off) if off is not None else None,
                        ctypes.c_long(off.size if off is not None else 1),
                        ctypes.c_double(eps), _ptr(y), ctypes.c_long(x.size))
    return y


def cast(x, dtype):
    """Cast.ts:27-95."""
    x = np.asarray(x)
    if dtype == "int32":
        if x.dtype == np.int32:
            return x.copy()
        if x.dtype == np.bool_ or x.dtype == np.uint8:
            return x.astype(np.int32)
        xf = _f32(x)
        y = np.empty(xf.shape, np.int32)
        lib().orc_cast_f32_i32(_ptr(xf), _ptr(y), ctypes.c_long(xf.size))
        return y
    if dtype == "bool":
        return (x != 0)
    if dtype == "float32":
        return x.astype(np.float32)
    raise ValueError("Error in Cast: failed to cast to %s" % dtype)


def gather(x, indices, axis=0, batch_dims=0):
    """GatherV2.ts:25-90: throws when an index is out of range (:36-46)."""
    x = np.asarray(x)
    indices = np.asarray(indices, dtype=np.int32)
    axis = axis % x.ndim
    dim = x.shape[axis]
    bad = (indices < 0) | (indices > dim - 1)
    if bad.any():
        raise ValueError("GatherV2: the index value %d is not in [0, %d]" %
                         (int(indices[bad][0]), dim - 1))
    if batch_dims == 0:
        return np.take(x, indices, axis=axis)
    out = [gather(x[i], indices[i], axis - 1, batch_dims - 1)
           for i in range(x.shape[0])]
    return np.stack(out, 0)


def transpose(x, perm):
    return np.ascontiguousarray(np.transpose(np.asarray(x), perm))


def dequantize(q, scale, min_val, dtype="float32"):
    """tfjs-core/src/io/io_utils.ts:221-227 (float32), :243-247 (int32)."""
    q = np.ascontiguousarray(q)
    is_u16 = int(q.dtype == np.uint16)
    assert q.dtype in (np.uint8, np.uint16)
    if dtype == "float32":
        out = np.empty(q.shape, np.float32)
        fn = lib().orc_dequant_f32
    else:
        out = np.empty(q.shape, np.int32)
        fn = lib().orc_dequant_i32
    fn(_ptr(q), is_u16, ctypes.c_double(scale), ctypes.c_double(min_val),
       _ptr(out), ctypes.c_long(q.size))
    return out


def decode_float16(q):
    """tfjs-core/src/io/io_utils.ts:720-741 (getFloat16Decoder) with the tables of
    :645-713: the table method of van der Zijp, "Fast Half Float Conversions" - a 2048-entry
    mantissa table (entries 1..1023 are the normalised subnormals, 1024..2047 the plain
    mantissas), a 64-entry exponent table and a 64-entry offset table indexed by the
    sign+exponent bits.  Returns float32 of the same shape as the uint16 input."""
    q = np.ascontiguousarray(q).view(np.uint16)
    mant = np.zeros(2048, np.uint64)
    for i in range(1, 1024):
        m, e = i << 13, 0
        while not (m & 0x00800000):
            e -= 0x00800000
            m <<= 1
        mant[i] = ((m & ~0x00800000) | ((e + 0x38800000) & 0xffffffff)) & 0xffffffff
    for i in range(1024, 2048):
        mant[i] = 0x38000000 + ((i - 1024) << 13)
    expo = np.zeros(64, np.uint64)
    expo[31], expo[32], expo[63] = 0x47800000, 0x80000000, 0xc7800000
    for i in range(1, 31):
        expo[i] = i << 23
    for i in range(33, 63):
        expo[i] = 0x80000000 + ((i - 32) << 23)
    off = np.full(64, 1024, np.int64)
    off[0] = off[32] = 0
    hi = (q >> 10).astype(np.int64)
    bits = (mant[off[hi] + (q & 0x3ff).astype(np.int64)] + expo[hi]) & 0xffffffff
    return bits.astype(np.uint32).view(np.float32).reshape(q.shape)
