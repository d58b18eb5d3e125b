"""Unary and broadcasting binary kernels, FusedBatchNorm, Cast.

Reference: tfjs-backend-cpu/src/utils/unary_utils.ts:34-79, binary_utils.ts:38-129,
binary_impl.ts:25-69 and the per-op files (Add.ts, Relu.ts, Erf.ts, ...);
BatchNorm.ts:23-90; Cast.ts:27-95.
"""
from .. import _cabi
from ..backend import (PendingConv, PendingDepthwise, PendingEw, PendingTile, TensorInfo)
from ..kernel_registry import KernelConfig
from ..util import assert_and_get_broadcast_shape, size_from_shape
from .common import BACKEND, assert_not_complex, dev, view

_I64 = _cabi.i64


def upcast_type(a, b):
    """tfjs-core/src/types.ts upcastType for the dtypes handled here."""
    order = {"bool": 0, "int32": 1, "float32": 2}
    return a if order[a] >= order[b] else b


def cast_impl(backend, x, dtype):
    """Cast.ts:27-95: widening casts are zero-copy in the reference; here only the
    same-dtype and bool->bool cases share the buffer because int32 and float32
    have different device representations."""
    if dtype not in _cabi.DTYPES:
        raise ValueError("Error in Cast: failed to cast %s to %s" % (x.dtype, dtype))
    if x.dtype == dtype:
        return view(backend, x, x.shape)
    out = backend.make_output(x.shape, dtype)
    try:
        backend.check(backend.lib.tfjs_cuda_cast(
            backend.ctx, _cabi.DTYPES[x.dtype], _cabi.DTYPES[dtype], dev(backend, x),
            size_from_shape(x.shape), dev(backend, out)))
    except Exception:
        backend.disposeData(out.dataId)
        raise
    return out


def unary_impl(backend, op, x, p0=0.0, p1=0.0):
    assert_not_complex(x, op)
    tmp = None
    if x.dtype != "float32":
        tmp = cast_impl(backend, x, "float32")
        x = tmp
    out = backend.make_output(x.shape, "float32")
    try:
        backend.check(backend.lib.tfjs_cuda_unary(
            backend.ctx, _cabi.UNARY_OPS[op], float(p0), float(p1), dev(backend, x),
            size_from_shape(x.shape), dev(backend, out)))
    except Exception:
        backend.disposeData(out.dataId)
        raise
    finally:
        if tmp is not None:
            backend.disposeData(tmp.dataId)
    return out


def binary_impl(backend, op, a, b, dtype=None):
    """binary_utils.ts:38-129: operands are upcast to a common dtype first."""
    assert_not_complex([a, b], op)
    out_dtype = dtype or upcast_type(a.dtype, b.dtype)
    if out_dtype == "bool":
        out_dtype = "int32"
    if op in ("RealDiv", "Pow", "SquaredDifference", "Prelu") and out_dtype != "float32":
        out_dtype = "float32" if op in ("RealDiv", "Prelu") else out_dtype
    tmp = []
    if a.dtype != out_dtype:
        a = cast_impl(backend, a, out_dtype)
        tmp.append(a)
    if b.dtype != out_dtype:
        b = cast_impl(backend, b, out_dtype)
        tmp.append(b)
    out_shape = assert_and_get_broadcast_shape(a.shape, b.shape)
    rank = len(out_shape)
    if rank > 6:
        raise ValueError("%s: rank %d is not supported by the CUDA backend" % (op, rank))
    pad = lambda s: [1] * (rank - len(s)) + list(s)
    out = backend.make_output(out_shape, out_dtype)
    try:
        backend.check(backend.lib.tfjs_cuda_binary(
            backend.ctx, _cabi.BINARY_OPS[op], _cabi.DTYPES[out_dtype], rank,
            dev(backend, a), _I64(pad(a.shape)), dev(backend, b), _I64(pad(b.shape)),
            dev(backend, out), _I64(out_shape)))
    except Exception:
        backend.disposeData(out.dataId)
        raise
    finally:
        for t in tmp:
            backend.disposeData(t.dataId)
    return out


def apply_activation(backend, x, activation, prelu=None, alpha=None):
    """tfjs-backend-cpu/src/utils/fused_utils.ts:29-49."""
    if activation in (None, "linear"):
        return view(backend, x, x.shape)
    if activation == "relu":
        return unary_impl(backend, "Relu", x)
    if activation == "elu":
        return unary_impl(backend, "Elu", x)
    if activation == "relu6":
        return unary_impl(backend, "Relu6", x)
    if activation == "prelu":
        return binary_impl(backend, "Prelu", x, prelu)
    if activation == "leakyrelu":
        return unary_impl(backend, "LeakyRelu", x, 0.2 if alpha is None else alpha)
    if activation == "sigmoid":
        return unary_impl(backend, "Sigmoid", x)
    raise ValueError("Activation %s has not been implemented for the CUDA backend." %
                     activation)


# ---------------------------------------------------------- deferred launches --
EW_BINARY = ("Add", "Sub", "Multiply", "RealDiv", "Maximum", "Minimum", "SquaredDifference")
EW_UNARY = ("Relu", "Relu6", "Elu", "Sigmoid", "Exp", "Sqrt", "Rsqrt", "Square", "Tanh", "Neg",
            "Erf", "Abs", "Log")


def _ew_operand(backend, info, leaves, leaf_shapes, ops, out_n, budget):
    """Reference to `info` inside the chain being built: a copy of its own pending
    chain when it has the result's size and has not been copied before (or is cheap to
    recompute), else a leaf."""
    pend = backend.pending_of(info.dataId)
    if (isinstance(pend, PendingEw) and size_from_shape(pend.shape) == out_n and
            (pend.consumed == 0 or pend.cheap()) and
            len(ops) + len(pend.ops) <= budget and
            len(set(leaves) | set(pend.leaves)) <= _cabi.EW_MAX_INPUTS):
        remap = []
        for leaf, shape in zip(pend.leaves, pend.leaf_shapes):
            if leaf not in leaves:
                leaves.append(leaf)
                leaf_shapes.append(shape)
            remap.append(leaves.index(leaf))
        base = len(ops)
        ref = lambda r: ("in", remap[r[1]]) if r[0] == "in" else ("op", base + r[1])
        for op in pend.ops:
            ops.append((op[0], ref(op[1]), ref(op[2])))
        pend.consumed += 1
        return ("op", len(ops) - 1), pend.desc
    if info.dataId not in leaves:
        leaves.append(info.dataId)
        leaf_shapes.append(list(info.shape))
    return ("in", leaves.index(info.dataId)), None


def deferred_elementwise(backend, name, a, b=None):
    """The float32 kernel `name` as a deferred launch joined to the pending chains of its
    operands; None when it has to run at once (other dtypes, empty or oversized tensors)."""
    if not backend.lazy_fusion or a.dtype != "float32" or (b is not None and b.dtype != "float32"):
        return None
    out_shape = list(a.shape) if b is None else assert_and_get_broadcast_shape(a.shape, b.shape)
    n = size_from_shape(out_shape)
    if n == 0 or len(out_shape) > 6:
        return None
    # launching a pending tensor walks its pending operands recursively: keep that shallow
    depth = 1
    for t in (a, b):
        if t is not None:
            pend = backend.pending_of(t.dataId)
            if isinstance(pend, PendingEw):
                if pend.depth >= 32:
                    backend.device_id(t.dataId)
                else:
                    depth = max(depth, pend.depth + 1)
    leaves, leaf_shapes, ops, descs = [], [], [], []
    budget = _cabi.EW_MAX_OPS - 2
    ra, da = _ew_operand(backend, a, leaves, leaf_shapes, ops, n, budget)
    rb, db = (ra, None) if b is None else _ew_operand(backend, b, leaves, leaf_shapes, ops, n,
                                                        budget)
    if len(leaves) > _cabi.EW_MAX_INPUTS:
        return None
    code = _cabi.BINARY_OPS[name] if b is not None else _cabi.EW_UNARY + _cabi.UNARY_OPS[name]
    ops.append((code, ra, rb))
    for d in (da, db):
        if d:
            descs.extend(d)
    ins = {}
    if ra[0] == "in":
        ins["a" if b is not None else "x"] = list(a.shape)
    if b is not None and rb[0] == "in" and rb != ra:
        ins["b"] = list(b.shape)
    descs.append({"name": name, "inputShapes": ins, "outputShapes": [out_shape], "attrs": {}})
    top = (code, a.dataId, list(a.shape), b.dataId if b is not None else None,
           list(b.shape) if b is not None else None)
    return backend.defer(out_shape, "float32",
                         PendingEw(leaves, leaf_shapes, ops, out_shape, descs, top, depth))


def _fold_activation(backend, name, x, attrs=None, other=None):
    """Relu / Relu6 over a pending convolution become the last step of its epilogue; so do
    the two ways tfjs-layers spells relu6 after a Relu: Minimum(6, .) (the Relu6 activation,
    tfjs-layers/src/activations.ts:83-89) and ClipByValue(., 0, 6) (the ReLU layer with
    maxValue 6, layers/advanced_activations.ts).  Returns the new pending tensor or None."""
    pend = backend.pending_of(x.dataId)
    if not isinstance(pend, (PendingConv, PendingDepthwise)) or x.dtype != "float32":
        return None
    act = None
    if name == "Relu" and pend.act == "linear":
        act = "relu"
    elif name == "Relu6" and pend.act in ("linear", "relu"):
        act = "relu6"
    elif name == "ClipByValue" and pend.act in ("linear", "relu"):
        if float(attrs["clipValueMin"]) == 0.0 and float(attrs["clipValueMax"]) == 6.0:
            act = "relu6"
    elif name == "Minimum" and pend.act == "relu" and other is not None:
        six = backend.host_values(other.dataId)
        if (other.dtype == "float32" and size_from_shape(other.shape) == 1 and six is not None
                and float(six[0]) == 6.0):
            act = "relu6"
    if act is None:
        return None
    desc = {"name": name, "inputShapes": {}, "outputShapes": [list(x.shape)], "attrs": {}}
    return backend.with_activation(x, act, desc)


def _depthwise_bias(backend, a, b):
    """Add of a pending depthwise convolution without a bias and a per-channel (or scalar)
    float32 operand, the biasAdd of tfjs-layers' DepthwiseConv2D: the convolution with that
    bias, still pending."""
    for conv, other in ((a, b), (b, a)):
        pend = backend.pending_of(conv.dataId)
        if not (isinstance(pend, PendingDepthwise) and pend.bias is None and
                pend.act == "linear" and other.dtype == "float32" and conv.dtype == "float32"):
            continue
        if backend.pending_of(other.dataId) is not None:
            continue
        channels = conv.shape[-1]
        n = size_from_shape(other.shape)
        per_channel = (n == channels and len(other.shape) <= len(conv.shape) and
                       other.shape[-1] == channels)
        if n != 1 and not per_channel:
            continue
        desc = {"name": "Add", "inputShapes": {"b": list(other.shape)},
                "outputShapes": [list(conv.shape)], "attrs": {}}
        return backend.defer(conv.shape, "float32",
                             pend.with_bias(other.dataId, 1 if n == 1 else channels, desc))
    return None


def _unary_config(name, p_from_attrs=None):
    def func(args):
        x = args["inputs"]["x"]
        backend = args["backend"]
        if x.dtype == "float32" and backend.lazy_fusion:
            if name in ("Relu", "Relu6", "ClipByValue"):
                out = _fold_activation(backend, name, x, args["attrs"])
                if out is not None:
                    return out
            if name in EW_UNARY:
                out = deferred_elementwise(backend, name, x)
                if out is not None:
                    return out
        p0, p1 = p_from_attrs(args["attrs"]) if p_from_attrs else (0.0, 0.0)
        return unary_impl(backend, name, x, p0, p1)
    return KernelConfig(name, BACKEND, func)


def _conv_residual(backend, a, b):
    """Add of a pending convolution and an equal-shape float32 tensor: the convolution with
    the other operand as its residual, still pending."""
    if not (a.dtype == "float32" and b.dtype == "float32" and list(a.shape) == list(b.shape)):
        return None
    desc = {"name": "Add", "inputShapes": {"b": list(b.shape)},
            "outputShapes": [list(a.shape)], "attrs": {}}
    for conv, other in ((a, b), (b, a)):
        pend = backend.pending_of(conv.dataId)
        if isinstance(pend, PendingConv) and pend.residual is None and pend.act == "linear":
            return backend.defer(a.shape, "float32", PendingConv(
                pend.params, pend.x, pend.filt, pend.bias, other.dataId, pend.desc + [desc]))
    return None


def _binary_config(name):
    def func(args):
        i = args["inputs"]
        backend = args["backend"]
        if name == "Prelu":
            return binary_impl(backend, name, i["x"], i["alpha"])
        if backend.lazy_fusion:
            out = None
            if name == "Add":
                out = _conv_residual(backend, i["a"], i["b"]) or \
                    _depthwise_bias(backend, i["a"], i["b"])
            elif name == "Minimum":
                out = _fold_activation(backend, name, i["a"], other=i["b"]) or \
                    _fold_activation(backend, name, i["b"], other=i["a"])
            if out is None and name in EW_BINARY:
                out = deferred_elementwise(backend, name, i["a"], i["b"])
            if out is not None:
                return out
        return binary_impl(backend, name, i["a"], i["b"])
    return KernelConfig(name, BACKEND, func)


def relu_int_aware(name):
    """Relu / Relu6 / Abs / Neg / Square on int32 keep int32 in the reference; the
    device kernels are float32, so int32 goes through Maximum/Minimum instead."""
    return _unary_config(name)


def fused_batch_norm(args):
    """BatchNorm.ts:23-90."""
    i, a, backend = args["inputs"], args["attrs"], args["backend"]
    x, mean, var = i["x"], i["mean"], i["variance"]
    scale, offset = i.get("scale"), i.get("offset")
    for t, nm in ((mean, "mean"), (var, "variance")):
        if len(t.shape) != 1 and list(t.shape) != list(x.shape)[-len(t.shape):]:
            pass  # the reference only asserts rank equality between parameters
    eps = a.get("varianceEpsilon")
    if eps is None:
        eps = 0.001
    n = size_from_shape(x.shape)
    rows_form = _batch_norm_rows(backend, x, mean, var, scale, offset, eps)
    if rows_form is not None:
        return rows_form
    out = backend.make_output(x.shape, "float32")
    try:
        backend.check(backend.lib.tfjs_cuda_batchnorm(
            backend.ctx, dev(backend, x), n, dev(backend, mean), size_from_shape(mean.shape),
            dev(backend, var), size_from_shape(var.shape),
            dev(backend, scale), size_from_shape(scale.shape) if scale is not None else 0,
            dev(backend, offset), size_from_shape(offset.shape) if offset is not None else 0,
            float(eps), dev(backend, out)))
    except Exception:
        backend.disposeData(out.dataId)
        raise
    return out


def _batch_norm_rows(backend, x, mean, var, scale, offset, eps):
    """tfjs-layers' LayerNormalization tiles the per-row moments and the per-column gamma /
    beta to x's shape and calls batchNorm on the tiles (layers/normalization.ts:578-622).
    When those Tile results are still pending, the kernel indexes the untiled tensors
    (tfjs_cuda_batchnorm_rows) and the tiles are never made.  None when the parameters are
    not of that form."""
    if x.dtype != "float32" or len(x.shape) < 1 or size_from_shape(x.shape) == 0:
        return None
    cols = x.shape[-1]
    rows = size_from_shape(x.shape) // cols if cols else 0
    row_shape, rank = list(x.shape[:-1]) + [1], len(x.shape)
    ids, modes, any_tile = [], [], False
    for t in (mean, var, scale, offset):
        if t is None:
            ids.append(None)
            modes.append(0)
            continue
        if t.dtype != "float32":
            return None
        pend = backend.pending_of(t.dataId)
        src_id, shape = t.dataId, list(t.shape)
        if isinstance(pend, PendingTile) and list(pend.shape) == list(x.shape):
            src_id, shape, any_tile = pend.src, list(pend.src_shape), True
        elif pend is not None:
            return None
        padded = [1] * (rank - len(shape)) + shape
        if len(padded) != rank:
            return None
        if size_from_shape(shape) == 1:
            mode = 4
        elif padded == list(x.shape):
            mode = 3
        elif padded == row_shape:
            mode = 2
        elif padded == [1] * (rank - 1) + [cols]:
            mode = 1
        else:
            return None
        ids.append(src_id)
        modes.append(mode)
    if not any_tile:
        return None
    out = backend.make_output(x.shape, "float32")
    try:
        d = [backend.device_id(i) if i is not None else 0 for i in ids]
        backend.check(backend.lib.tfjs_cuda_batchnorm_rows(
            backend.ctx, dev(backend, x), rows, cols, d[0], modes[0], d[1], modes[1], d[2],
            modes[2], d[3], modes[3], float(eps), dev(backend, out)))
    except Exception:
        backend.disposeData(out.dataId)
        raise
    return out


def cast(args):
    return cast_impl(args["backend"], args["inputs"]["x"], args["attrs"]["dtype"])


CONFIGS = (
    [_unary_config(n) for n in ("Relu", "Relu6", "Elu", "Sigmoid", "Exp", "Sqrt", "Rsqrt",
                                "Square", "Tanh", "Neg", "Erf", "Abs", "Log")] +
    [_unary_config("LeakyRelu", lambda a: (a.get("alpha", 0.2), 0.0)),
     _unary_config("ClipByValue", lambda a: (a["clipValueMin"], a["clipValueMax"]))] +
    [_binary_config(n) for n in ("Add", "Sub", "Multiply", "RealDiv", "Maximum", "Minimum",
                                 "Pow", "SquaredDifference", "Prelu")] +
    [KernelConfig("FusedBatchNorm", BACKEND, fused_batch_norm),
     KernelConfig("Cast", BACKEND, cast)]
)
