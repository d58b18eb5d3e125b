"""CudaBackend: the host half of `tfjs-backend-cuda`.

Python mirror of the TypeScript class a Node build would ship.  It implements the
KernelBackend contract (tfjs-core/src/backends/backend.ts:100-156) with the
semantics of the reference CPU backend (tfjs-backend-cpu/src/backend_cpu.ts):

  write / move / read / readSync / disposeData / refCount / incRef / decRef /
  numDataIds / memory / time / floatPrecision / dispose

and owns one `tfjs_cuda_ctx` (one GPU).  DataIds are fresh objects, as in the
reference (`const dataId = {id: this.nextDataId()}`, backend_cpu.ts:58).

Small tensors written from the host stay host-resident and are uploaded only
when a kernel first consumes them.  The graph executor reads axis / shape / perm
Const tensors with dataSync() inside its node loop
(tfjs-converter/src/operations/executors/utils.ts:55); with this rule those
reads never touch the CUDA stream.

Deferred launches.  A FusedConv2D with a linear activation and the float32 unary / binary
elementwise kernels return a tensor whose launch is pending; it is launched when the
tensor is first read or consumed by another kind of kernel.  An Add that consumes a
pending convolution, and a Relu / Relu6 that consumes that, fold into the convolution's
epilogue (`tfjs_cuda_fused_conv2d_residual`), which removes the separate Add and Relu
passes of a residual block; chains of elementwise kernels (the decomposed LayerNorm and
GELU of a transformer graph) become one `tfjs_cuda_fused_elementwise` pass.  Every step still rounds to fp32
in the order of the separate kernels, so results do not change.  The WebGL backend
defers work behind the same KernelBackend contract (uploads and packing happen on
first use, tfjs-backend-webgl/src/backend_webgl.ts uploadToGPU).  Set
TFJS_CUDA_NO_LAZY_FUSION=1 to launch every kernel eagerly.
"""
import ctypes
import os
import time as _time
from ctypes import byref, c_float, c_int32, c_uint64, c_void_p

import numpy as np

from . import _cabi
from ._cabi import CudaError

NP_DTYPES = {"float32": np.float32, "int32": np.int32, "bool": np.uint8}
HOST_RESIDENT_BYTES = 4096  # keep a host copy of tensors up to this size


class DataId(object):
    """Opaque key object; identity is the key (a WeakMap key in tfjs)."""
    __slots__ = ("id", "__weakref__")
    _next = 0

    def __init__(self):
        DataId._next += 1
        self.id = DataId._next

    def __repr__(self):
        return "DataId(%d)" % self.id


class TensorInfo(object):
    """tfjs-core/src/tensor_info.ts: {dataId, shape, dtype}."""
    __slots__ = ("dataId", "shape", "dtype")

    def __init__(self, dataId, shape, dtype):
        self.dataId = dataId
        self.shape = [int(s) for s in shape]
        self.dtype = dtype

    @property
    def size(self):
        n = 1
        for s in self.shape:
            n *= s
        return n

    def __repr__(self):
        return "TensorInfo(%r, %s, %s)" % (self.dataId, self.shape, self.dtype)


class _Record(object):
    __slots__ = ("dev", "nbytes", "dtype", "ref", "host", "pending", "held")

    def __init__(self, dev, nbytes, dtype, ref, host):
        self.dev = dev        # device buffer id, 0 = not uploaded / not launched yet
        self.nbytes = nbytes
        self.dtype = dtype
        self.ref = ref
        self.host = host      # numpy copy for small host-written tensors
        self.pending = None   # PendingConv / PendingAdd until the launch happens
        self.held = 0         # how many of `ref` belong to pending launches


class PendingConv(object):
    """A FusedConv2D (bias fused, linear activation) not launched yet, optionally with
    the operand of the Add that consumed it and the activation that followed (`act`:
    linear, relu or relu6, applied last)."""
    __slots__ = ("params", "x", "filt", "bias", "residual", "desc", "act", "dw_folded")

    def __init__(self, params, x, filt, bias, residual, desc, act="linear"):
        self.params, self.x, self.filt, self.bias = params, x, filt, bias
        self.residual = residual
        self.desc = desc      # profile records of the kernels folded into this launch
        self.act = act
        self.dw_folded = False

    def deps(self):
        return [d for d in (self.x, self.filt, self.bias, self.residual) if d is not None]

    def with_act(self, act, desc):
        return PendingConv(self.params, self.x, self.filt, self.bias, self.residual,
                           self.desc + [desc], act)

    def _launch_with_depthwise(self, backend, out_dev, post_act):
        """If the input is a depthwise convolution that is still pending and this is the
        1x1 convolution behind it (the projection of an inverted-residual block), both run
        as one launch and the depthwise result is never written.  False when the pair is
        not of that form or the library does not take the shapes."""
        rec = backend.data.get(self.x)
        dw = rec.pending if rec is not None else None
        p = self.params
        if not (backend.fuse_depthwise_project and isinstance(dw, PendingDepthwise)):
            return False
        d = dw.params
        if not (d.filter_h == 3 and d.filter_w == 3 and d.stride_h == d.stride_w and d.stride_h in (1, 2) and
                d.dilation_h == 1 and d.dilation_w == 1 and d.out_c == d.in_c and
                d.in_c % 4 == 0 and dw.act in ("linear", "relu", "relu6") and
                p.filter_h == 1 and p.filter_w == 1 and p.stride_h == 1 and p.stride_w == 1 and
                p.pad_top == 0 and p.pad_left == 0 and p.out_h == p.in_h and
                p.out_w == p.in_w and p.out_c % 4 == 0 and 8 <= p.out_c <= 512 and
                (self.residual is not None or post_act == "linear" or
                 p.activation == _cabi.ACTIVATIONS["linear"])):
            return False
        dp = _cabi.Conv2DParams.from_buffer_copy(d)
        dp.activation = _cabi.ACTIVATIONS[dw.act]
        pp = p
        post = _cabi.ACTIVATIONS["linear"]
        if self.residual is not None:
            post = _cabi.ACTIVATIONS[post_act]
        elif post_act != "linear":
            pp = _cabi.Conv2DParams.from_buffer_copy(p)
            pp.activation = _cabi.ACTIVATIONS[post_act]
        # Operands that are pending themselves launch now, and such a launch may, further
        # down, need this very depthwise result and materialise it (a block's output feeds
        # both the next block and that block's shortcut).  So the shortcut and the weights
        # come first, then the depthwise convolution is looked at again, and its input, which
        # it keeps alive, comes last.
        ids = [backend.device_id(t) if t is not None else 0
               for t in (dw.filt, dw.bias, self.filt, self.bias, self.residual)]
        if rec.pending is not dw:
            return False
        rc = backend.lib.tfjs_cuda_fused_depthwise_project(
            backend.ctx, byref(dp), byref(pp), backend.device_id(dw.x), ids[0], ids[1], ids[2],
            ids[3], ids[4], post, out_dev)
        if rc == _cabi.UNSUPPORTED:
            return False
        backend.check(rc)
        if not self.dw_folded:
            # profile records: the depthwise kernels join this launch, and the convolution
            # no longer reads its input from memory
            own = dict(self.desc[0])
            own["inputShapes"] = {k: v for k, v in own["inputShapes"].items() if k != "x"}
            self.desc[:] = [dict(t) for t in dw.desc] + [own] + self.desc[1:]
            self.dw_folded = True
        return True

    def launch(self, backend, out_dev, post_act):
        lib, p = backend.lib, self.params
        post_act = self.act if post_act == "linear" else post_act
        if self._launch_with_depthwise(backend, out_dev, post_act):
            return
        bias = backend.device_id(self.bias) if self.bias is not None else 0
        if self.residual is None:
            if post_act != "linear":
                p = _cabi.Conv2DParams.from_buffer_copy(p)
                p.activation = _cabi.ACTIVATIONS[post_act]
            backend.check(lib.tfjs_cuda_fused_conv2d(
                backend.ctx, byref(p), backend.device_id(self.x), backend.device_id(self.filt),
                bias, 0, out_dev))
        else:
            backend.check(lib.tfjs_cuda_fused_conv2d_residual(
                backend.ctx, byref(p), backend.device_id(self.x), backend.device_id(self.filt),
                bias, 0, backend.device_id(self.residual), _cabi.ACTIVATIONS[post_act],
                out_dev))


class PendingDepthwise(object):
    """A DepthwiseConv2dNative / FusedDepthwiseConv2D with a linear activation not launched
    yet.  tfjs-layers' DepthwiseConv2D layer issues the convolution, then Add with the bias
    reshaped to [1, 1, 1, C], then the activation as kernels of their own
    (tfjs-layers/src/layers/convolutional_depthwise.ts:154-169); here the bias of that Add
    and a following Relu / Relu6 (spelled Relu then Minimum(6, .) or ClipByValue(., 0, 6) by
    the Relu6 activation and the ReLU layer) join the convolution's launch, which applies
    them with the same fp32 roundings."""
    __slots__ = ("params", "x", "filt", "bias", "desc", "act")

    def __init__(self, params, x, filt, bias, desc, act="linear"):
        self.params, self.x, self.filt, self.bias = params, x, filt, bias
        self.desc, self.act = desc, act

    def deps(self):
        return [d for d in (self.x, self.filt, self.bias) if d is not None]

    def with_bias(self, bias, bias_len, desc):
        p = _cabi.Conv2DParams.from_buffer_copy(self.params)
        p.bias_len = bias_len
        return PendingDepthwise(p, self.x, self.filt, bias, self.desc + [desc], self.act)

    def with_act(self, act, desc):
        return PendingDepthwise(self.params, self.x, self.filt, self.bias, self.desc + [desc], act)

    def launch(self, backend, out_dev, post_act):
        p = _cabi.Conv2DParams.from_buffer_copy(self.params)
        p.activation = _cabi.ACTIVATIONS[self.act if post_act == "linear" else post_act]
        backend.check(backend.lib.tfjs_cuda_fused_depthwise_conv2d(
            backend.ctx, byref(p), backend.device_id(self.x), backend.device_id(self.filt),
            backend.device_id(self.bias) if self.bias is not None else 0, 0, out_dev))


class PendingMatMul(object):
    """A _FusedMatMul (or its heads-split form) with a fused bias, not launched yet.  When
    it is launched, the other products still pending on the same `a` operand with the same
    dimensions (the query, key and value projections of an attention layer) go with it in
    one `tfjs_cuda_fused_matmul_group` launch; each member's result is the one its own
    launch would give."""
    __slots__ = ("params", "a", "b", "bias", "heads", "desc", "key")

    def __init__(self, params, a, b, bias, heads, desc):
        self.params, self.a, self.b, self.bias = params, a, b, bias
        self.heads = heads    # None, or (layout, rows_or_heads, head_dim) of the permuted store
        self.desc = desc
        self.key = (bytes(params), heads, bias is None)

    def deps(self):
        return [d for d in (self.a, self.b, self.bias) if d is not None]

    def launch(self, backend, out_dev, post_act):
        lib = backend.lib
        bias = backend.device_id(self.bias) if self.bias is not None else 0
        if self.heads is None:
            backend.check(lib.tfjs_cuda_fused_matmul(
                backend.ctx, byref(self.params), backend.device_id(self.a),
                backend.device_id(self.b), bias, 0, out_dev))
        else:
            backend.check(lib.tfjs_cuda_fused_matmul_heads(
                backend.ctx, byref(self.params), backend.device_id(self.a),
                backend.device_id(self.b), bias, 0, self.heads[0], self.heads[1], self.heads[2],
                out_dev))


class PendingTile(object):
    """A Tile not launched yet.  A consumer that can index the untiled tensor itself (the
    batch normalisation behind tfjs-layers' LayerNormalization, which tiles the moments and
    gamma / beta to the input's shape) reads `src` directly and the tile never exists; any
    other consumer makes it materialise."""
    __slots__ = ("src", "src_shape", "reps", "shape", "dtype", "desc")

    def __init__(self, src, src_shape, reps, shape, dtype, desc):
        self.src, self.src_shape, self.reps = src, [int(v) for v in src_shape], list(reps)
        self.shape, self.dtype, self.desc = [int(v) for v in shape], dtype, desc

    def deps(self):
        return [self.src]

    def launch(self, backend, out_dev, post_act):
        from .kernels import movement
        movement.tile_into(backend, TensorInfo(self.src, self.src_shape, self.dtype), self.reps,
                           self.shape, out_dev)


class PendingEw(object):
    """A chain of float32 elementwise kernels not launched yet.

    `leaves` are the tensors the chain reads (dataIds, with their shapes); `ops` are
    (opcode, a, b) in execution order, operands being ("in", k) for leaf k or ("op", j)
    for the result of op j; the last op's result is the tensor.  Opcodes are the C ABI's:
    binary op numbers, or 32 + unary op number.  `depth` counts the pending tensors
    stacked below this one (bounded by the kernel funcs, since launching walks them
    recursively)."""
    __slots__ = ("leaves", "leaf_shapes", "ops", "shape", "desc", "consumed", "top", "depth")

    def __init__(self, leaves, leaf_shapes, ops, shape, desc, top, depth=1):
        self.depth = depth
        self.leaves, self.leaf_shapes, self.ops = leaves, leaf_shapes, ops
        self.shape, self.desc = [int(v) for v in shape], desc
        self.consumed = 0   # how many later chains took a copy of this one
        # the kernel call that created this tensor: (opcode, a dataId, a shape, b dataId or
        # None, b shape).  A chain the library has no fused kernel for is launched as this
        # one kernel on its operand tensors, which launches their chains the same way, so
        # nothing is ever computed twice.
        self.top = top

    def deps(self):
        out = list(self.leaves)
        for d in (self.top[1], self.top[3]):
            if d is not None and d not in out:
                out.append(d)
        return out

    def cheap(self):
        """True when every leaf is smaller than the result (broadcast scalars, rows and
        biases only): recomputing such a chain inside each consumer costs no memory pass."""
        n = size_from_shape(self.shape)
        return len(self.ops) <= 2 and all(size_from_shape(s) < n for s in self.leaf_shapes)

    # ------------------------------------------------------------- launching --
    def _leaf_mode(self, shape):
        """(mode, period, aux) of a leaf relative to the result's flat index, or None."""
        out = self.shape
        n, m = size_from_shape(out), size_from_shape(shape)
        rank = len(out)
        sh = [1] * (rank - len(shape)) + [int(v) for v in shape]
        if len(sh) != rank:
            return None
        if m == 1:
            return (_cabi.EW_SCALAR, 1, 0)
        if m == n:
            return (_cabi.EW_FULL, 0, 0)
        d = 0
        while d < rank and sh[d] == 1:
            d += 1
        if sh[d:] == out[d:]:
            return (_cabi.EW_PERIODIC, m, 0)
        if rank >= 1 and sh[-1] == 1 and sh[:-1] == out[:-1]:
            return (_cabi.EW_ROW, 0, 0)
        p = 0
        while p < rank and sh[p] == out[p]:
            p += 1
        q = p
        while q < rank and sh[q] == 1:
            q += 1
        if 0 < p < q < rank and sh[q:] == out[q:]:
            inner = size_from_shape(out[q:])
            return (_cabi.EW_BATCHED, inner, inner * size_from_shape(out[p:q]))
        return None

    def launch(self, backend, out_dev, post_act):
        assert post_act == "linear"
        ops = self.ops
        n = size_from_shape(self.shape)
        modes = [self._leaf_mode(s) for s in self.leaf_shapes]
        if len(ops) == 1 or n >= (1 << 31) or any(m is None for m in modes):
            return self._launch_top(backend, out_dev)
        # Add (+ Relu / Relu6) of two full tensors has a kernel of its own
        if (len(self.leaves) == 2 and all(m[0] == _cabi.EW_FULL for m in modes) and
                ops[0][0] == _cabi.BINARY_OPS["Add"] and
                {ops[0][1], ops[0][2]} == {("in", 0), ("in", 1)} and len(ops) == 2 and
                ops[1][0] in (_cabi.EW_UNARY + _cabi.UNARY_OPS["Relu"],
                              _cabi.EW_UNARY + _cabi.UNARY_OPS["Relu6"])):
            act = "relu" if ops[1][0] == _cabi.EW_UNARY + _cabi.UNARY_OPS["Relu"] else "relu6"
            return backend.check(backend.lib.tfjs_cuda_add_activation(
                backend.ctx, _cabi.ACTIVATIONS[act], backend.device_id(self.leaves[0]),
                backend.device_id(self.leaves[1]), n, out_dev))
        # canonical order (commutative operands sorted by structure, ops in evaluation
        # order from the result, leaves numbered by first use), then the library's
        # catalogue of straight-line chain kernels; other chains run kernel by kernel
        c_ops, leaf_order = _canonical_program(ops, [m[0] for m in modes])
        prog = _cabi.EwProgram()
        prog.n_inputs, prog.n_ops, prog.n = len(leaf_order), len(c_ops), n
        prog.cols = max(int(self.shape[-1]) if self.shape else 1, 1)
        slot = lambda ref: ref[1] if ref[0] == "in" else len(leaf_order) + ref[1]
        for j, (code, a, b) in enumerate(c_ops):
            prog.ops[j].opcode, prog.ops[j].a, prog.ops[j].b = code, slot(a), slot(b)
        signature = tuple((code, slot(a), slot(b)) for code, a, b in c_ops)
        known = backend.ew_catalogue.get(signature)
        if known is None:
            yes = c_int32()
            backend.check(backend.lib.tfjs_cuda_fused_elementwise_catalogued(
                backend.ctx, byref(prog), byref(yes)))
            known = backend.ew_catalogue[signature] = bool(yes.value)
        if not known:
            return self._launch_top(backend, out_dev)
        for k, leaf in enumerate(leaf_order):
            prog.input_id[k] = backend.device_id(self.leaves[leaf])
            prog.input_mode[k], prog.input_period[k], prog.input_aux[k] = modes[leaf]
        backend.check(backend.lib.tfjs_cuda_fused_elementwise(backend.ctx, byref(prog), out_dev))

    def _launch_top(self, backend, out_dev):
        """The separate kernel of the call that made this tensor, on its operand tensors
        (whose own pending launches happen first)."""
        code, a, a_shape, b, b_shape = self.top
        lib = backend.lib
        # this launch covers the last kernel of the chain only (what the profile records)
        ins = {"a" if b is not None else "x": list(a_shape)}
        if b is not None:
            ins["b"] = list(b_shape)
        self.desc[:] = [dict(self.desc[-1], inputShapes=ins)]
        if code >= _cabi.EW_UNARY:
            return backend.check(lib.tfjs_cuda_unary(
                backend.ctx, code - _cabi.EW_UNARY, 0.0, 0.0, backend.device_id(a),
                size_from_shape(self.shape), out_dev))
        rank = len(self.shape)
        pad = lambda sh: _cabi.i64([1] * (rank - len(sh)) + [int(v) for v in sh])
        backend.check(lib.tfjs_cuda_binary(
            backend.ctx, code, _cabi.DTYPES["float32"], rank, backend.device_id(a), pad(a_shape),
            backend.device_id(b), pad(b_shape), out_dev, _cabi.i64(self.shape)))


_EW_COMMUTATIVE = frozenset(_cabi.BINARY_OPS[n] for n in
                            ("Add", "Multiply", "Maximum", "Minimum", "SquaredDifference"))


def _canonical_program(ops, leaf_modes):
    """(ops, leaf order) of an elementwise chain in canonical form: operands of
    commutative ops ordered by a structural key, ops emitted in evaluation order from the
    result, leaves numbered by first use, a value used twice emitted once.  ops in and
    out are (opcode, a, b, ...) with operand references ("in", k) / ("op", j)."""
    keys = {}

    def key(ref):
        k = keys.get(ref)
        if k is None:
            if ref[0] == "in":
                k = "L%d" % leaf_modes[ref[1]]
            else:
                code, a, b = ops[ref[1]][:3]
                if code >= _cabi.EW_UNARY:
                    k = "(%d %s)" % (code, key(a))
                else:
                    ka, kb = key(a), key(b)
                    if code in _EW_COMMUTATIVE and kb < ka:
                        ka, kb = kb, ka
                    k = "(%d %s %s)" % (code, ka, kb)
            keys[ref] = k
        return k

    out, leaf_order, done = [], [], {}

    def emit(ref):
        r = done.get(ref)
        if r is None:
            if ref[0] == "in":
                leaf_order.append(ref[1])
                r = ("in", len(leaf_order) - 1)
            else:
                code, a, b = ops[ref[1]][:3]
                if code >= _cabi.EW_UNARY:
                    ra = rb = emit(a)
                else:
                    if code in _EW_COMMUTATIVE and key(b) < key(a):
                        a, b = b, a
                    ra, rb = emit(a), emit(b)
                out.append((code, ra, rb))
                r = ("op", len(out) - 1)
            done[ref] = r
        return r

    emit(("op", len(ops) - 1))
    return out, leaf_order


class PendingRead(object):
    """Result of CudaBackend.read: the Promise of backend.read in tfjs."""
    __slots__ = ("backend", "ticket", "values", "dtype")

    def __init__(self, backend, ticket, values, dtype):
        self.backend, self.ticket, self.values, self.dtype = backend, ticket, values, dtype

    def wait(self):
        if self.ticket:
            ticket, self.ticket = self.ticket, 0
            self.backend.check(self.backend.lib.tfjs_cuda_read_wait(self.backend.ctx, ticket))
        return self.values.astype(np.bool_) if self.dtype == "bool" else self.values


def size_from_shape(shape):
    n = 1
    for s in shape:
        n *= int(s)
    return n


class CudaBackend(object):
    """One instance per GPU (`device_ordinal`)."""

    def __init__(self, device_ordinal=0):
        self.lib = _cabi.load()
        ctx = c_void_p()
        rc = self.lib.tfjs_cuda_create(int(device_ordinal), byref(ctx))
        if rc != _cabi.OK:
            raise CudaError(rc, "tfjs_cuda_create(device %d) failed with status "
                            "%d: no usable sm_100a GPU" % (device_ordinal, rc))
        self.ctx = ctx
        self.device_ordinal = device_ordinal
        self.data = {}        # DataId -> _Record
        self._pinned = []
        self._hidden = 0      # records kept alive only by pending launches
        self.lazy_fusion = os.environ.get("TFJS_CUDA_NO_LAZY_FUSION", "0") in ("", "0")
        # a pending 3x3 depthwise convolution consumed by a 1x1 convolution runs inside that
        # convolution's launch (TFJS_CUDA_NO_DW_PROJECT=1 keeps the two launches)
        self.fuse_depthwise_project = os.environ.get("TFJS_CUDA_NO_DW_PROJECT", "0") in ("", "0")
        # products that share their first operand launch together (TFJS_CUDA_NO_MATMUL_GROUP=1
        # launches each on its own); dataId of `a` -> dataIds of the pending products on it
        self.math_mode = "tf32"
        self.group_matmuls = os.environ.get("TFJS_CUDA_NO_MATMUL_GROUP", "0") in ("", "0")
        self._matmuls_on = {}
        self.profiler = None  # the engine, while it profiles (told about deferred launches)
        self.ew_catalogue = {}  # chain signature -> the library has a kernel for it
        self._log_depth = 0     # nesting of launch_log(True)

    # ------------------------------------------------------------ plumbing --
    def check(self, rc):
        if rc != _cabi.OK:
            msg = self.lib.tfjs_cuda_last_error(self.ctx)
            raise CudaError(rc, msg.decode() if msg else "status %d" % rc)

    def _alloc(self, nbytes):
        out = c_int32()
        self.check(self.lib.tfjs_cuda_alloc(self.ctx, int(nbytes), byref(out)))
        return out.value

    def floatPrecision(self):
        return 32

    def epsilon(self):
        return 1e-7

    # -------------------------------------------------- KernelBackend: data --
    def write(self, values, shape, dtype):
        """backend_cpu.ts:52-71."""
        dataId = DataId()
        self.move(dataId, values, shape, dtype, 1)
        return dataId

    def move(self, dataId, values, shape, dtype, refCount):
        """backend_cpu.ts:119-123."""
        if dtype not in NP_DTYPES:
            raise ValueError("tfjs-backend-cuda: dtype %s is not supported" % dtype)
        n = size_from_shape(shape)
        arr = None
        if values is not None:
            arr = np.ascontiguousarray(np.asarray(values).astype(NP_DTYPES[dtype],
                                                                 copy=False)).reshape(-1)
            if arr.size != n:
                raise ValueError("write: %d values for shape %s" % (arr.size, list(shape)))
        nbytes = n * np.dtype(NP_DTYPES[dtype]).itemsize
        rec = _Record(0, nbytes, dtype, refCount, None)
        if arr is not None and nbytes <= HOST_RESIDENT_BYTES:
            rec.host = arr.copy()
        else:
            rec.dev = self._alloc(nbytes)
            if arr is not None and nbytes:
                self.check(self.lib.tfjs_cuda_write(self.ctx, rec.dev,
                                                    arr.ctypes.data_as(c_void_p), nbytes))
        self.data[dataId] = rec

    def make_output(self, shape, dtype):
        """Allocate an uninitialised device tensor for a kernel result
        (makeTensorInfo, backend_cpu.ts:83-95)."""
        nbytes = size_from_shape(shape) * np.dtype(NP_DTYPES[dtype]).itemsize
        dataId = DataId()
        self.data[dataId] = _Record(self._alloc(nbytes), nbytes, dtype, 1, None)
        return TensorInfo(dataId, shape, dtype)

    # ---------------------------------------------------- deferred launches --
    def _adjust(self, rec, dref, dheld):
        """Change a record's reference counts, tracking whether only pending launches
        keep it alive (such records are not reported by numDataIds)."""
        was = rec.held > 0 and rec.ref <= rec.held
        rec.ref += dref
        rec.held += dheld
        now = rec.held > 0 and rec.ref <= rec.held
        if was != now:
            self._hidden += 1 if now else -1

    def defer(self, shape, dtype, pending):
        """Output tensor of a kernel whose launch is deferred; the inputs stay alive
        until the launch happened or the output was disposed."""
        nbytes = size_from_shape(shape) * np.dtype(NP_DTYPES[dtype]).itemsize
        dataId = DataId()
        rec = _Record(0, nbytes, dtype, 1, None)
        rec.pending = pending
        for d in pending.deps():
            self._adjust(self.data[d], 1, 1)
        self.data[dataId] = rec
        if isinstance(pending, PendingMatMul):
            if len(self._matmuls_on) > 64:     # forget operands whose products are all gone
                self._matmuls_on = {a: ids for a, ids in self._matmuls_on.items()
                                    if any(self._still_pending_matmul(i) for i in ids)}
            ids = [i for i in self._matmuls_on.get(pending.a, []) if self._still_pending_matmul(i)]
            self._matmuls_on[pending.a] = ids + [dataId]
        return TensorInfo(dataId, shape, dtype)

    def _still_pending_matmul(self, dataId):
        rec = self.data.get(dataId)
        return rec is not None and isinstance(rec.pending, PendingMatMul)

    def _resolve_matmul_group(self, rec, pending):
        """Launches `pending` together with the other products pending on the same operand
        (same dimensions, layout and bias kind).  False when there is no such product or the
        library does not take the group; nothing has been launched then."""
        ids = self._matmuls_on.get(pending.a, [])
        mates = [self.data[i] for i in ids if self._still_pending_matmul(i)]
        mates = [m for m in mates if m is not rec and m.pending.key == pending.key][:3]
        if not (self.group_matmuls and mates):
            return False
        # operands that are pending launch first; the group is what is still pending then
        a_dev = self.device_id(pending.a)
        for m in mates:
            if m.pending is not None:
                for t in (m.pending.b, m.pending.bias):
                    if t is not None:
                        self.device_id(t)
        for t in (pending.b, pending.bias):
            if t is not None:
                self.device_id(t)
        mates = [m for m in mates if isinstance(m.pending, PendingMatMul)]
        if rec.pending is not pending or not mates:
            return False
        members = [rec] + mates
        devs = []
        try:
            for m in members:
                devs.append(self._alloc(m.nbytes))
            n = len(members)
            arr = c_int32 * n
            b_ids = arr(*[self.device_id(m.pending.b) for m in members])
            bias_ids = arr(*[self.device_id(m.pending.bias) if m.pending.bias is not None else 0
                             for m in members])
            heads = pending.heads or (0, 0, 0)
            descs = [d for m in members for d in m.pending.desc]

            def launch():
                return self.lib.tfjs_cuda_fused_matmul_group(
                    self.ctx, byref(pending.params), a_dev, n, b_ids, bias_ids,
                    heads[0], heads[1], heads[2], arr(*devs))
            rc = launch() if self.profiler is None else \
                self.profiler.deferred_launch(descs, launch, False)
            if rc == _cabi.UNSUPPORTED:
                for d in devs:
                    self.lib.tfjs_cuda_free(self.ctx, d)
                return False
            self.check(rc)
        except Exception:
            for d in devs:
                self.lib.tfjs_cuda_free(self.ctx, d)
            raise
        for m, d in zip(members, devs):
            done, m.pending = m.pending, None
            m.dev = d
            self._release(done)
        return True

    def pending_of(self, dataId):
        return self.data[dataId].pending

    def _release(self, pending):
        for d in pending.deps():
            rec = self.data[d]
            self._adjust(rec, -1, -1)
            if rec.ref <= 0:
                self._drop(d, rec)

    def _launch(self, pending, dev, post_act, fold_into_caller):
        if self.profiler is None:
            return pending.launch(self, dev, post_act)
        # operands that are themselves pending launch inside, as records of their own
        return self.profiler.deferred_launch(
            pending.desc, lambda: pending.launch(self, dev, post_act), fold_into_caller)

    def _resolve(self, rec):
        pending = rec.pending
        if isinstance(pending, PendingMatMul) and self._resolve_matmul_group(rec, pending):
            return
        if rec.pending is not pending:      # launched meanwhile, by an operand's own launch
            return
        dev = self._alloc(rec.nbytes)
        try:
            self._launch(pending, dev, "linear", False)
        except Exception:
            self.lib.tfjs_cuda_free(self.ctx, dev)
            raise
        rec.dev = dev
        rec.pending = None
        self._release(pending)

    def with_activation(self, info, act, desc):
        """The pending convolution behind `info` with `act` (relu / relu6) as the last step
        of its epilogue, as a new pending tensor.  `info` itself stays pending: if another
        kernel consumes it later it is launched again, without the activation."""
        pending = self.data[info.dataId].pending
        return self.defer(info.shape, "float32", pending.with_act(act, desc))

    def device_id(self, dataId):
        """Device buffer id of a tensor; launches a pending producer or uploads a
        host-resident tensor first."""
        rec = self.data[dataId]
        if rec.pending is not None:
            self._resolve(rec)
        elif rec.dev == 0:
            rec.dev = self._alloc(rec.nbytes)
            if rec.nbytes:
                self.check(self.lib.tfjs_cuda_write(
                    self.ctx, rec.dev, rec.host.ctypes.data_as(c_void_p), rec.nbytes))
        return rec.dev

    def host_values(self, dataId):
        """Host copy if the tensor is host-resident, else None (no sync)."""
        return self.data[dataId].host

    def readSync(self, dataId):
        """backend_cpu.ts:129-144: the only blocking call besides time()."""
        rec = self.data[dataId]
        if rec.pending is not None:
            self._resolve(rec)
        if rec.host is not None:
            out = rec.host.copy()
        else:
            out = np.empty(rec.nbytes // np.dtype(NP_DTYPES[rec.dtype]).itemsize,
                           NP_DTYPES[rec.dtype])
            self.check(self.lib.tfjs_cuda_read(self.ctx, rec.dev,
                                               out.ctypes.data_as(c_void_p), rec.nbytes))
        return out.astype(np.bool_) if rec.dtype == "bool" else out

    def read(self, dataId, into=None):
        """backend.read(dataId): Promise (backend.ts:104).  Queues the device-to-host
        copy behind the kernels launched so far and returns a PendingRead at once;
        `.wait()` blocks until the bytes are there.  `into` is an optional (ideally
        pinned) numpy array that receives them."""
        rec = self.data[dataId]
        if rec.pending is not None:
            self._resolve(rec)
        npdt = NP_DTYPES[rec.dtype]
        if rec.host is not None:
            if into is None:
                into = rec.host.copy()
            else:
                into.reshape(-1)[:] = rec.host
            return PendingRead(self, 0, into, rec.dtype)
        if into is None:
            into = np.empty(rec.nbytes // np.dtype(npdt).itemsize, npdt)
        ticket = c_int32()
        self.check(self.lib.tfjs_cuda_read_begin(self.ctx, rec.dev, into.ctypes.data_as(c_void_p),
                                                 rec.nbytes, byref(ticket)))
        return PendingRead(self, ticket.value, into, rec.dtype)

    def read_into(self, dataId, host_array):
        """readSync into caller-provided (ideally pinned) memory."""
        rec = self.data[dataId]
        if rec.pending is not None:
            self._resolve(rec)
        if rec.host is not None:
            host_array.reshape(-1)[:] = rec.host
            return
        self.check(self.lib.tfjs_cuda_read(self.ctx, rec.dev,
                                           host_array.ctypes.data_as(c_void_p), rec.nbytes))

    def disposeData(self, dataId, force=False):
        """backend_cpu.ts:176-193: true iff the memory was released."""
        rec = self.data.get(dataId)
        if rec is None:
            return False
        self._adjust(rec, -1, 0)
        if rec.ref > 0 and (not force or rec.held > 0):
            return False
        self._drop(dataId, rec)
        return True

    def _drop(self, dataId, rec):
        if rec.held > 0 and rec.ref <= rec.held:
            self._hidden -= 1
        del self.data[dataId]
        if rec.dev:
            self.check(self.lib.tfjs_cuda_free(self.ctx, rec.dev))
        if rec.pending is not None:
            pending, rec.pending = rec.pending, None
            self._release(pending)

    def refCount(self, dataId):
        rec = self.data.get(dataId)
        return rec.ref - rec.held if rec is not None else 0

    def incRef(self, dataId):
        self._adjust(self.data[dataId], 1, 0)

    def decRef(self, dataId):
        rec = self.data.get(dataId)
        if rec is not None:
            self._adjust(rec, -1, 0)

    def numDataIds(self):
        return len(self.data) - self._hidden

    def memory(self):
        """tfjs-core/src/engine.ts:959-974 merges this into tf.memory()."""
        vals = [c_uint64() for _ in range(4)]
        self.check(self.lib.tfjs_cuda_memory(self.ctx, *[byref(v) for v in vals]))
        return {"unreliable": False, "numBytesInGPU": vals[0].value,
                "numBytesInGPUAllocated": vals[1].value,
                "poolHighWater": vals[2].value, "numDeviceBuffers": vals[3].value}

    def time(self, f):
        """backend.time(f) -> BackendTimingInfo (backend.ts:26-30): {kernelMs, wallMs,
        getExtraProfileInfo} with CUDA events on the stream; the extra information names
        the kernel instantiations the library launched inside f."""
        t0 = _time.perf_counter()
        nested = self._log_depth > 0
        self.launch_log(True)
        try:
            self.check(self.lib.tfjs_cuda_time_begin(self.ctx))
            f()
            ms = c_float()
            self.check(self.lib.tfjs_cuda_time_end(self.ctx, byref(ms)))
            info = self.launch_log_take() if not nested else ""
        finally:
            self.launch_log(False)
        return {"kernelMs": ms.value, "wallMs": (_time.perf_counter() - t0) * 1e3,
                "getExtraProfileInfo": lambda: info}

    def launch_log(self, enable):
        """Turns the library's launch log on or off (calls nest)."""
        if enable:
            self._log_depth += 1
            if self._log_depth == 1:
                self.check(self.lib.tfjs_cuda_launch_log(self.ctx, 1))
        else:
            self._log_depth -= 1
            if self._log_depth == 0:
                self.check(self.lib.tfjs_cuda_launch_log(self.ctx, 0))

    def launch_log_take(self):
        """Text naming the kernel instantiations launched since the last take."""
        buf = ctypes.create_string_buffer(4096)
        self.check(self.lib.tfjs_cuda_launch_log_take(self.ctx, buf, 4096, None))
        return buf.value.decode()

    def event_record(self, slot):
        self.check(self.lib.tfjs_cuda_event_record(self.ctx, int(slot)))

    def event_elapsed(self, slot_begin, slot_end):
        ms = c_float()
        self.check(self.lib.tfjs_cuda_event_elapsed(self.ctx, int(slot_begin), int(slot_end),
                                                    byref(ms)))
        return ms.value

    def timerAvailable(self):
        return True

    def sync(self):
        self.check(self.lib.tfjs_cuda_sync(self.ctx))

    def set_math_mode(self, mode):
        """'tf32' (tensor cores) or 'fp32' (SIMT fp32 FMA)."""
        self.check(self.lib.tfjs_cuda_set_math_mode(
            self.ctx, {"tf32": _cabi.MATH_TF32, "fp32": _cabi.MATH_FP32}[mode]))
        self.math_mode = mode

    # ------------------------------------------------ whole-step capture / replay --
    def high_water_reset(self):
        self.check(self.lib.tfjs_cuda_high_water_reset(self.ctx))

    def copy(self, src_dataId, dst_dataId):
        """Device-to-device copy of a whole tensor, in stream order."""
        nbytes = self.data[src_dataId].nbytes
        self.check(self.lib.tfjs_cuda_copy(self.ctx, self.device_id(src_dataId),
                                           self.device_id(dst_dataId), nbytes))

    def capture_begin(self, arena_bytes):
        self.check(self.lib.tfjs_cuda_capture_begin(self.ctx, int(arena_bytes)))

    def capture_end(self, abandon=False):
        """Graph id of the captured step; raises CudaError (UNSUPPORTED) when the capture
        had to be discarded."""
        graph = c_int32()
        self.check(self.lib.tfjs_cuda_capture_end(self.ctx, 1 if abandon else 0, byref(graph)))
        return graph.value

    def graph_launch(self, graph):
        self.check(self.lib.tfjs_cuda_graph_launch(self.ctx, int(graph)))

    def graph_destroy(self, graph):
        self.check(self.lib.tfjs_cuda_graph_destroy(self.ctx, int(graph)))

    def launch_count(self):
        v = c_uint64()
        self.check(self.lib.tfjs_cuda_launch_count(self.ctx, byref(v)))
        return v.value

    def flush_l2(self):
        self.check(self.lib.tfjs_cuda_flush_l2(self.ctx))

    def pinned_empty(self, shape, dtype):
        """numpy array over pinned host memory owned by this backend."""
        n = size_from_shape(shape)
        npdt = np.dtype(NP_DTYPES[dtype] if isinstance(dtype, str) else dtype)
        nbytes = max(n * npdt.itemsize, 1)
        ptr = c_void_p()
        self.check(self.lib.tfjs_cuda_host_alloc(self.ctx, nbytes, byref(ptr)))
        self._pinned.append(ptr)
        buf = (ctypes.c_uint8 * nbytes).from_address(ptr.value)
        return np.frombuffer(buf, dtype=npdt, count=n).reshape(shape)

    def write_from(self, host_array, shape, dtype):
        """write() that always goes to the device straight from `host_array`
        (use with pinned_empty for asynchronous H2D)."""
        n = size_from_shape(shape)
        nbytes = n * np.dtype(NP_DTYPES[dtype]).itemsize
        dataId = DataId()
        dev = c_int32()
        # copy-stream upload: overlaps whatever is already queued on the compute stream
        self.check(self.lib.tfjs_cuda_upload(self.ctx, host_array.ctypes.data_as(c_void_p),
                                             nbytes, byref(dev)))
        self.data[dataId] = _Record(dev.value, nbytes, dtype, 1, None)
        return dataId

    def dispose(self):
        if self.ctx:
            for ptr in self._pinned:
                self.lib.tfjs_cuda_host_free(self.ctx, ptr)
            self._pinned = []
            self.lib.tfjs_cuda_destroy(self.ctx)
            self.ctx = None
            self.data = {}

    def __del__(self):
        try:
            self.dispose()
        except Exception:
            pass
