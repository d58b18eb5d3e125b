"""Softmax, Sum, Mean, Max, ArgMax.

Reference: tfjs-backend-cpu/src/kernels/Softmax.ts:29-77, Sum.ts:28-90,
Mean.ts:25-53, Max.ts:28-72, ArgMax.ts:24-71.  The reference transposes the
reduced axes innermost; here contiguous reduced axes are reduced in place over an
[outer, reduce, inner] view and only a non-contiguous set is transposed first.
"""
import numpy as np

from .. import _cabi
from ..kernel_registry import KernelConfig
from ..util import (compute_out_and_reduce_shapes, expand_shape_to_keep_dim,
                    get_axes_permutation, get_inner_most_axes, parse_axis_param,
                    size_from_shape)
from .common import BACKEND, assert_not_complex, dev
from . import elementwise, movement


def _collapse(backend, x, axes):
    """Returns (tensor, outer, reduce, inner, temporaries) with the reduced axes
    forming one contiguous run."""
    rank = len(x.shape)
    axes = sorted(set(axes))
    tmp = []
    contiguous = all(axes[i] + 1 == axes[i + 1] for i in range(len(axes) - 1))
    if not contiguous:
        perm = get_axes_permutation(axes, rank)
        x = movement.transpose_impl(backend, x, perm)
        tmp.append(x)
        axes = get_inner_most_axes(len(axes), rank)
    if not axes:
        return x, size_from_shape(x.shape), 1, 1, tmp
    outer = size_from_shape(x.shape[:axes[0]])
    red = size_from_shape(x.shape[axes[0]:axes[-1] + 1])
    inner = size_from_shape(x.shape[axes[-1] + 1:])
    return x, outer, red, inner, tmp


def reduce_impl(backend, op, x, axis, keep_dims):
    assert_not_complex(x, op.lower())
    axes = parse_axis_param(axis, x.shape)
    out_shape, _ = compute_out_and_reduce_shapes(x.shape, axes)
    tmp = []
    if x.dtype != "float32":
        x = elementwise.cast_impl(backend, x, "float32")
        tmp.append(x)
    xt, outer, red, inner, t2 = _collapse(backend, x, axes)
    tmp += t2
    shape = expand_shape_to_keep_dim(out_shape, sorted(axes)) if keep_dims else out_shape
    out = backend.make_output(shape, "float32")
    try:
        backend.check(backend.lib.tfjs_cuda_reduce(
            backend.ctx, _cabi.REDUCE_OPS[op], dev(backend, xt), outer, red, inner,
            dev(backend, out)))
    except Exception:
        backend.disposeData(out.dataId)
        raise
    finally:
        for t in tmp:
            backend.disposeData(t.dataId)
    return out


def _sum(args):
    a = args["attrs"]
    x = args["inputs"]["x"]
    out = reduce_impl(args["backend"], "Sum", x, a.get("axis"), a.get("keepDims", False))
    if x.dtype in ("int32", "bool"):
        # Sum.ts:57: the result dtype is upcast(x.dtype, 'int32').
        r = elementwise.cast_impl(args["backend"], out, "int32")
        args["backend"].disposeData(out.dataId)
        return r
    return out


def _mean(args):
    a = args["attrs"]
    return reduce_impl(args["backend"], "Mean", args["inputs"]["x"], a.get("axis"),
                       a.get("keepDims", False))


def _max(args):
    a = args["attrs"]
    x = args["inputs"]["x"]
    out = reduce_impl(args["backend"], "Max", x, a.get("reductionIndices"),
                      a.get("keepDims", False))
    if x.dtype == "int32":
        r = elementwise.cast_impl(args["backend"], out, "int32")
        args["backend"].disposeData(out.dataId)
        return r
    return out


def _argmax(args):
    backend, x = args["backend"], args["inputs"]["x"]
    assert_not_complex(x, "argMax")
    axes = parse_axis_param(args["attrs"].get("axis", 0), x.shape)[:1]
    out_shape, _ = compute_out_and_reduce_shapes(x.shape, axes)
    tmp = []
    if x.dtype != "float32":
        x = elementwise.cast_impl(backend, x, "float32")
        tmp.append(x)
    outer = size_from_shape(x.shape[:axes[0]])
    red = x.shape[axes[0]]
    inner = size_from_shape(x.shape[axes[0] + 1:])
    out = backend.make_output(out_shape, "int32")
    try:
        backend.check(backend.lib.tfjs_cuda_argmax(backend.ctx, dev(backend, x), outer, red,
                                                   inner, dev(backend, out)))
    except Exception:
        backend.disposeData(out.dataId)
        raise
    finally:
        for t in tmp:
            backend.disposeData(t.dataId)
    return out


def _softmax(args):
    backend, logits = args["backend"], args["inputs"]["logits"]
    dim = args["attrs"].get("dim", -1)
    rank = len(logits.shape)
    if dim == -1:
        dim = rank - 1
    if dim != rank - 1:
        raise ValueError("Softmax along a non-last dimension is not yet supported. "
                         "Logits was rank %d and dim was %d" % (rank, dim))
    cols = logits.shape[-1]
    rows = size_from_shape(logits.shape[:-1])
    out = backend.make_output(logits.shape, "float32")
    try:
        backend.check(backend.lib.tfjs_cuda_softmax(backend.ctx, dev(backend, logits), rows,
                                                    cols, dev(backend, out)))
    except Exception:
        backend.disposeData(out.dataId)
        raise
    return out


def softmax_mask_rows(x_shape, mask_shape):
    """rows_per_mask for a mask that broadcasts against x over whole rows: the mask equals x
    on the last axis and on a (possibly empty) run of leading axes and is 1 in between.
    None when it broadcasts any other way."""
    rank = len(x_shape)
    m = [1] * (rank - len(mask_shape)) + list(mask_shape)
    if len(m) != rank or rank == 0 or m[-1] != x_shape[-1]:
        return None
    lead = 0
    while lead < rank - 1 and m[lead] == x_shape[lead]:
        lead += 1
    if any(d != 1 for d in m[lead:rank - 1]):
        return None
    return max(size_from_shape(list(x_shape[lead:rank - 1])), 1)


def _softmax_scaled_masked(args):
    """softmax(x * scale + mask) over the last axis in one launch (the scaled, masked scores
    of an attention layer; graph_model.fuse_softmax_inputs)."""
    backend, inp, at = args["backend"], args["inputs"], args["attrs"]
    x, mask = inp["logits"], inp.get("mask")
    scale = at.get("scale")
    cols = x.shape[-1]
    rows = size_from_shape(x.shape[:-1])
    rpm = 1
    if mask is not None:
        rpm = softmax_mask_rows(x.shape, mask.shape)
        if rpm is None or mask.dtype != "float32":
            raise ValueError("_SoftmaxScaledMasked: mask %s does not broadcast over rows of %s"
                             % (mask.shape, x.shape))
    out = backend.make_output(x.shape, "float32")
    try:
        backend.check(backend.lib.tfjs_cuda_softmax_scaled_masked(
            backend.ctx, dev(backend, x), rows, cols, int(scale is not None),
            float(np.float32(scale if scale is not None else 1.0)), dev(backend, mask), rpm,
            dev(backend, out)))
    except Exception:
        backend.disposeData(out.dataId)
        raise
    return out


def _fused_attention(args):
    """softmax(q k^T * scale + mask) v for q, k, v of shape [B, H, S, D], stored [B, S, H, D]:
    one launch for the two batched products, the scaled, masked softmax between them and
    the transpose behind them (graph_model.fuse_attention).  Raises CudaError(UNSUPPORTED)
    for shapes the library does not take; nothing has been launched then."""
    backend, inp, at = args["backend"], args["inputs"], args["attrs"]
    q, k, v, mask = inp["q"], inp["k"], inp["v"], inp.get("mask")
    scale = at.get("scale")
    if len(q.shape) != 4 or list(k.shape) != list(q.shape) or list(v.shape) != list(q.shape) \
            or any(t.dtype != "float32" for t in (q, k, v)):
        raise _cabi.CudaError(_cabi.UNSUPPORTED, "_FusedAttention: q, k, v of one 4-D shape")
    B, H, S, D = [int(d) for d in q.shape]
    upm = 1
    if mask is not None:
        rpm = softmax_mask_rows([B, H, S, S], mask.shape) if mask.dtype == "float32" else None
        if rpm is None or rpm % S != 0:
            raise _cabi.CudaError(_cabi.UNSUPPORTED,
                                  "_FusedAttention: mask %s is not one row per head" % (mask.shape,))
        upm = rpm // S
    out = backend.make_output([B, S, H, D], "float32")
    try:
        backend.check(backend.lib.tfjs_cuda_fused_attention(
            backend.ctx, dev(backend, q), dev(backend, k), dev(backend, v), dev(backend, mask),
            int(scale is not None), float(np.float32(scale if scale is not None else 1.0)),
            B, H, S, D, upm, dev(backend, out)))
    except Exception:
        backend.disposeData(out.dataId)
        raise
    return out


def layer_norm_supported(x_shape, gamma_shape, beta_shape):
    """Shapes the one-launch layer normalisation takes: rows of a multiple of 4 up to 1024
    floats, gamma and beta one value per column."""
    if not x_shape:
        return False
    cols = x_shape[-1]
    return (cols % 4 == 0 and 0 < cols <= 1024 and size_from_shape(gamma_shape) == cols and
            size_from_shape(beta_shape) == cols and
            (not gamma_shape or gamma_shape[-1] == cols) and
            (not beta_shape or beta_shape[-1] == cols))


def _fused_layer_norm(args):
    """((x - mean) * rsqrt(var + epsilon)) * gamma + beta over the last axis, the subgraph
    the graph executor matches (graph_model.fuse_layer_norms), in one launch; with
    `residual`, of Add(x, residual)."""
    backend, inp = args["backend"], args["inputs"]
    x, gamma, beta = inp["x"], inp["gamma"], inp["beta"]
    residual = inp.get("residual")
    if residual is not None and (list(residual.shape) != list(x.shape) or
                                 residual.dtype != "float32"):
        raise ValueError("_FusedLayerNorm: residual %s does not have the shape of x %s" %
                         (residual.shape, x.shape))
    if not layer_norm_supported(x.shape, gamma.shape, beta.shape):
        raise ValueError("_FusedLayerNorm: unsupported shapes %s %s %s" %
                         (x.shape, gamma.shape, beta.shape))
    cols = x.shape[-1]
    rows = size_from_shape(x.shape[:-1])
    out = backend.make_output(x.shape, "float32")
    try:
        backend.check(backend.lib.tfjs_cuda_layer_norm(
            backend.ctx, dev(backend, x), dev(backend, residual), dev(backend, gamma),
            dev(backend, beta), rows, cols,
            float(np.float32(args["attrs"]["epsilon"])), dev(backend, out)))
    except Exception:
        backend.disposeData(out.dataId)
        raise
    return out


CONFIGS = [
    KernelConfig("Sum", BACKEND, _sum),
    KernelConfig("Mean", BACKEND, _mean),
    KernelConfig("Max", BACKEND, _max),
    KernelConfig("ArgMax", BACKEND, _argmax),
    KernelConfig("Softmax", BACKEND, _softmax),
    KernelConfig("_FusedLayerNorm", BACKEND, _fused_layer_norm),
    KernelConfig("_SoftmaxScaledMasked", BACKEND, _softmax_scaled_masked),
    KernelConfig("_FusedAttention", BACKEND, _fused_attention),
]
