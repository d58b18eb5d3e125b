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

Deferred launches.  A FusedConv2D with a linear activation and a same-shape float32
Add return a tensor whose launch is pending; it is launched when the tensor is first
read or consumed by another kernel.  An Add that consumes a pending convolution, and a
Relu / Relu6 that consumes either, fold into the producer's epilogue instead
(`tfjs_cuda_fused_conv2d_residual`, `tfjs_cuda_add_activation`), which removes the
separate Add and Relu passes of a residual block.  Every step still rounds to fp32
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
    the operand of the Add that consumed it."""
    __slots__ = ("params", "x", "filt", "bias", "residual", "desc")

    def __init__(self, params, x, filt, bias, residual, desc):
        self.params, self.x, self.filt, self.bias = params, x, filt, bias
        self.residual = residual
        self.desc = desc      # profile records of the kernels folded into this launch

    def deps(self):
        return [d for d in (self.x, self.filt, self.bias, self.residual) if d is not None]

    def launch(self, backend, out_dev, post_act):
        lib, p = backend.lib, self.params
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


class PendingAdd(object):
    """A same-shape float32 Add not launched yet."""
    __slots__ = ("a", "b", "n", "desc")

    def __init__(self, a, b, n, desc):
        self.a, self.b, self.n, self.desc = a, b, n, desc

    def deps(self):
        return [self.a, self.b]

    def launch(self, backend, out_dev, post_act):
        backend.check(backend.lib.tfjs_cuda_add_activation(
            backend.ctx, _cabi.ACTIVATIONS[post_act], backend.device_id(self.a),
            backend.device_id(self.b), self.n, out_dev))


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
        self.profiler = None  # the engine, while it profiles (told about deferred launches)

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
        return TensorInfo(dataId, shape, dtype)

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
        # operands that are themselves pending launch first, as records of their own
        for d in pending.deps():
            self.device_id(d)
        return self.profiler.deferred_launch(
            pending.desc, lambda: pending.launch(self, dev, post_act), fold_into_caller)

    def _resolve(self, rec):
        pending = rec.pending
        dev = self._alloc(rec.nbytes)
        try:
            self._launch(pending, dev, "linear", False)
        except Exception:
            self.lib.tfjs_cuda_free(self.ctx, dev)
            raise
        rec.dev = dev
        rec.pending = None
        self._release(pending)

    def launch_pending(self, info, post_act):
        """Launch the pending producer of `info` with `post_act` (relu / relu6) folded
        into its epilogue and return the activated tensor.  `info` itself stays
        pending: if another kernel consumes it later it is launched again, without
        the activation."""
        pending = self.data[info.dataId].pending
        out = self.make_output(info.shape, "float32")
        try:
            self._launch(pending, self.data[out.dataId].dev, post_act, True)
        except Exception:
            self.disposeData(out.dataId)
            raise
        return out

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
        """backend.time(f) -> {kernelMs, wallMs} with CUDA events on the stream."""
        t0 = _time.perf_counter()
        self.check(self.lib.tfjs_cuda_time_begin(self.ctx))
        f()
        ms = c_float()
        self.check(self.lib.tfjs_cuda_time_end(self.ctx, byref(ms)))
        return {"kernelMs": ms.value, "wallMs": (_time.perf_counter() - t0) * 1e3}

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
