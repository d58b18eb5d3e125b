"""Reshape, Identity, ExpandDims (zero-copy), Transpose, GatherV2, Concat, Slice,
PadV2, Tile, Pack.

Reference: tfjs-backend-cpu/src/kernels/Reshape.ts:22-53, Identity.ts:22-30,
ExpandDims.ts, Transpose.ts:25-48, GatherV2.ts:25-90, Concat.ts:29-103, Slice.ts,
PadV2.ts, Tile.ts, Pack.ts.
"""
from ctypes import byref, c_int64

import numpy as np

from .. import _cabi
from ..kernel_registry import KernelConfig
from ..util import (collect_gather_op_shape_info, compute_strides, parse_axis_param,
                    size_from_shape)
from .common import BACKEND, dev, view

_I64, _I32 = _cabi.i64, _cabi.i32


def _elem_bytes(dtype):
    return 1 if dtype == "bool" else 4


def reshape_impl(backend, x, shape):
    """Reshape.ts:22-53, with the -1 inference of util.inferFromImplicitShape."""
    shape = [int(s) for s in shape]
    x_size = size_from_shape(x.shape)
    if shape.count(-1) > 1:
        raise ValueError("Shapes can only have 1 implicit size.")
    if -1 in shape:
        known = 1
        for s in shape:
            if s != -1:
                known *= s
        if known == 0 or x_size % known:
            raise ValueError("The implicit shape can't be a fractional number. Got %d / %d"
                             % (x_size, known))
        shape[shape.index(-1)] = x_size // known
    if size_from_shape(shape) != x_size:
        raise ValueError("The new shape (%s) has %d elements and the old shape (%s) has %d "
                         "elements. The new shape and old shape must have the same number "
                         "of elements." % (shape, size_from_shape(shape), x.shape, x_size))
    return view(backend, x, shape)


def transpose_impl(backend, x, perm):
    rank = len(x.shape)
    perm = [int(p) for p in perm]
    if rank > 6:
        raise ValueError("Transpose: rank %d is not supported by the CUDA backend" % rank)
    if sorted(perm) != list(range(rank)):
        raise ValueError("Error in transpose: rank of input %d must match length of perm %s."
                         % (rank, perm))
    out_shape = [x.shape[p] for p in perm]
    out = backend.make_output(out_shape, x.dtype)
    try:
        backend.check(backend.lib.tfjs_cuda_transpose(
            backend.ctx, _elem_bytes(x.dtype), rank, dev(backend, x), _I64(x.shape),
            _I32(perm), dev(backend, out)))
    except Exception:
        backend.disposeData(out.dataId)
        raise
    return out


def copy_strided(backend, x, x_off, x_strides, x_wrap, out, o_off, o_strides, extent):
    rank = len(extent)
    if rank > 6:
        raise ValueError("rank %d is not supported by the CUDA backend" % rank)
    backend.check(backend.lib.tfjs_cuda_copy_strided(
        backend.ctx, _elem_bytes(x.dtype), rank, _I64(extent), dev(backend, x), int(x_off),
        _I64(x_strides), _I64(x_wrap), dev(backend, out), int(o_off), _I64(o_strides)))


def slice_impl(backend, x, begin, size):
    """Slice.ts with slice_util.parseSliceParams."""
    rank = len(x.shape)
    begin = [int(b) for b in (begin if isinstance(begin, (list, tuple, np.ndarray)) else
                              [begin] + [0] * (rank - 1))]
    if size is None:
        size = [-1] * rank
    size = [int(s) for s in (size if isinstance(size, (list, tuple, np.ndarray)) else
                             [size] + [-1] * (rank - 1))]
    begin = begin + [0] * (rank - len(begin))
    size = size + [-1] * (rank - len(size))
    size = [x.shape[d] - begin[d] if size[d] < 0 else size[d] for d in range(rank)]
    for d in range(rank):
        if begin[d] < 0 or begin[d] + size[d] > x.shape[d]:
            raise ValueError("Error in slice%dD: begin[%d] + size[%d] (%d) would overflow "
                             "input.shape[%d] (%d)" % (rank, d, d, begin[d] + size[d], d,
                                                       x.shape[d]))
    out = backend.make_output(size, x.dtype)
    if size_from_shape(size):
        xs = compute_strides(x.shape)
        off = sum(b * s for b, s in zip(begin, xs))
        try:
            copy_strided(backend, x, off, xs, x.shape if rank else [], out, 0,
                         compute_strides(size), size)
        except Exception:
            backend.disposeData(out.dataId)
            raise
    return out


def concat_impl(backend, tensors, axis):
    """Concat.ts:29-103: empty inputs are dropped, shapes must agree off-axis."""
    axis = parse_axis_param(axis, tensors[0].shape)[0]
    shapes = [t.shape for t in tensors]
    rank = len(shapes[0])
    for s in shapes:
        if len(s) != rank:
            raise ValueError("Error in concat%dD: rank of tensors must be the same." % rank)
        for d in range(rank):
            if d != axis and s[d] != shapes[0][d]:
                raise ValueError("Error in concat%dD: Shape of tensors (%s) does not match "
                                 "the shape of the rest (%s) along the non-concatenated axis."
                                 % (rank, s, shapes[0]))
    out_shape = list(shapes[0])
    out_shape[axis] = sum(s[axis] for s in shapes)
    live = [t for t in tensors if size_from_shape(t.shape) > 0]
    if len(live) == 1 and list(live[0].shape) == out_shape:
        return view(backend, live[0], out_shape)
    dtype = tensors[0].dtype
    out = backend.make_output(out_shape, dtype)
    os_ = compute_strides(out_shape)
    pos = 0
    try:
        for t in tensors:
            if size_from_shape(t.shape):
                copy_strided(backend, t, 0, compute_strides(t.shape), t.shape, out,
                             pos * os_[axis], os_, t.shape)
            pos += t.shape[axis]
    except Exception:
        backend.disposeData(out.dataId)
        raise
    return out


def _reshape(args):
    return reshape_impl(args["backend"], args["inputs"]["x"], args["attrs"]["shape"])


def _identity(args):
    x = args["inputs"]["x"]
    return view(args["backend"], x, x.shape)


def _expand_dims(args):
    x = args["inputs"]["input"]
    dim = int(args["attrs"]["dim"])
    rank = len(x.shape)
    if dim > rank:
        raise ValueError("Axis must be <= rank of the tensor")
    if dim < 0:
        if -(rank + 1) > dim:
            raise ValueError("Axis must be in the interval [%d, %d]" % (-(rank + 1), rank))
        dim = rank + dim + 1
    shape = list(x.shape)
    shape.insert(dim, 1)
    return view(args["backend"], x, shape)


def _transpose(args):
    return transpose_impl(args["backend"], args["inputs"]["x"], args["attrs"]["perm"])


def _gather(args):
    """GatherV2.ts:25-90.  The index range check (:36-46) runs on the host when the
    indices are host-resident, otherwise on the device."""
    i, a, backend = args["inputs"], args["attrs"], args["backend"]
    x, indices = i["x"], i["indices"]
    axis = parse_axis_param(a.get("axis", 0), x.shape)[0]
    batch_dims = a.get("batchDims", 0) or 0
    if indices.dtype != "int32":
        raise ValueError("GatherV2: indices must be int32, got %s" % indices.dtype)
    info = collect_gather_op_shape_info(x.shape, indices.shape, axis, batch_dims)
    dim = x.shape[axis]
    host_idx = backend.host_values(indices.dataId)
    check_on_device = 1
    if host_idx is not None:
        bad = host_idx[(host_idx < 0) | (host_idx > dim - 1)]
        if bad.size:
            raise ValueError("GatherV2: the index value %d is not in [0, %d]" %
                             (int(bad[0]), dim - 1))
        check_on_device = 0
    n_idx = size_from_shape(indices.shape) // max(info["batchSize"], 1)
    out = backend.make_output(info["outputShape"], x.dtype)
    bad_index = c_int64(-1)
    try:
        backend.check(backend.lib.tfjs_cuda_gather(
            backend.ctx, _elem_bytes(x.dtype), dev(backend, x), dev(backend, indices),
            info["batchSize"], info["outerSize"], info["dimSize"], info["sliceSize"], n_idx,
            dev(backend, out), check_on_device, byref(bad_index)))
    except Exception as e:
        backend.disposeData(out.dataId)
        raise ValueError(str(e))
    return out


def _concat(args):
    return concat_impl(args["backend"], list(args["inputs"]), args["attrs"].get("axis", 0)) \
        if isinstance(args["inputs"], (list, tuple)) else \
        concat_impl(args["backend"], [args["inputs"][k] for k in sorted(args["inputs"],
                                                                         key=lambda s: int(s))],
                    args["attrs"].get("axis", 0))


def _slice(args):
    return slice_impl(args["backend"], args["inputs"]["x"], args["attrs"]["begin"],
                      args["attrs"].get("size"))


def _pad(args):
    """PadV2.ts: out = constant everywhere, x copied at offset `paddings[d][0]`."""
    backend, x = args["backend"], args["inputs"]["x"]
    paddings = args["attrs"]["paddings"]
    const = args["attrs"].get("constantValue", 0) or 0
    out_shape = [int(p[0]) + s + int(p[1]) for p, s in zip(paddings, x.shape)]
    out = backend.make_output(out_shape, x.dtype)
    n = size_from_shape(out_shape)
    try:
        if x.dtype == "float32":
            bits = int(np.float32(const).view(np.uint32))
        elif x.dtype == "int32":
            bits = int(np.int32(const).view(np.uint32))
        else:
            bits = int(bool(const))
        backend.check(backend.lib.tfjs_cuda_fill(backend.ctx, _elem_bytes(x.dtype), bits,
                                                 dev(backend, out), n))
        if size_from_shape(x.shape):
            os_ = compute_strides(out_shape)
            off = sum(int(p[0]) * s for p, s in zip(paddings, os_))
            copy_strided(backend, x, 0, compute_strides(x.shape), x.shape, out, off, os_,
                         x.shape)
    except Exception:
        backend.disposeData(out.dataId)
        raise
    return out


def _tile(args):
    """Tile.ts: out[loc] = x[loc mod x.shape]."""
    backend, x = args["backend"], args["inputs"]["x"]
    reps = [int(r) for r in args["attrs"]["reps"]]
    if len(reps) != len(x.shape):
        raise ValueError("Error in transpose: rank of input %d must match length of reps %s."
                         % (len(x.shape), reps))
    out_shape = [s * r for s, r in zip(x.shape, reps)]
    if (backend.lazy_fusion and x.dtype == "float32" and size_from_shape(out_shape) and
            len(out_shape) <= 6 and backend.pending_of(x.dataId) is None):
        # Deferred: a batch normalisation that can index the untiled tensor never needs it
        from ..backend import PendingTile
        desc = {"name": "Tile", "inputShapes": {"x": list(x.shape)},
                "outputShapes": [out_shape], "attrs": {}}
        return backend.defer(out_shape, x.dtype,
                             PendingTile(x.dataId, x.shape, reps, out_shape, x.dtype, [desc]))
    out = backend.make_output(out_shape, x.dtype)
    if size_from_shape(out_shape):
        try:
            tile_into(backend, x, reps, out_shape, dev(backend, out))
        except Exception:
            backend.disposeData(out.dataId)
            raise
    return out


def tile_into(backend, x, reps, out_shape, out_dev):
    """The tile of x written to the device buffer out_dev."""
    rank = len(out_shape)
    if rank > 6:
        raise ValueError("rank %d is not supported by the CUDA backend" % rank)
    backend.check(backend.lib.tfjs_cuda_copy_strided(
        backend.ctx, _elem_bytes(x.dtype), rank, _I64(out_shape), dev(backend, x), 0,
        _I64(compute_strides(x.shape)), _I64(x.shape), out_dev, 0,
        _I64(compute_strides(out_shape))))


def _pack(args):
    """Pack.ts: expandDims each input along `axis`, then concat."""
    backend = args["backend"]
    tensors = list(args["inputs"]) if isinstance(args["inputs"], (list, tuple)) else \
        [args["inputs"][k] for k in sorted(args["inputs"], key=lambda s: int(s))]
    axis = int(args["attrs"].get("axis", 0))
    if len(tensors) == 1:
        return _expand_dims({"inputs": {"input": tensors[0]}, "attrs": {"dim": axis},
                             "backend": backend})
    shape = list(tensors[0].shape)
    if axis < 0:
        axis += len(shape) + 1
    shape.insert(axis, 1)
    views = [view(backend, t, shape) for t in tensors]
    try:
        return concat_impl(backend, views, axis)
    finally:
        for v in views:
            backend.disposeData(v.dataId)


CONFIGS = [
    KernelConfig("Reshape", BACKEND, _reshape),
    KernelConfig("Identity", BACKEND, _identity),
    KernelConfig("ExpandDims", BACKEND, _expand_dims),
    KernelConfig("Transpose", BACKEND, _transpose),
    KernelConfig("GatherV2", BACKEND, _gather),
    KernelConfig("Concat", BACKEND, _concat),
    KernelConfig("Slice", BACKEND, _slice),
    KernelConfig("PadV2", BACKEND, _pad),
    KernelConfig("Tile", BACKEND, _tile),
    KernelConfig("Pack", BACKEND, _pack),
]
