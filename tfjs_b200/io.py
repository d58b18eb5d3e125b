"""Weight (de)coding for graph models.

`decode_weights` is the drop-in for `io.decodeWeights`
(tfjs-core/src/io/io_utils.ts:119-135, :185-292): GraphModel receives the io
namespace as a constructor argument and calls `this.io.decodeWeights`
(tfjs-converter/src/executor/graph_model.ts:104-107, :177), so a backend can
supply one that leaves uint8 / uint16 affine-quantised weights quantised on the
way to the GPU and dequantises them there, once, at load time.

`quantize_weights` restates the converter's affine quantisation
(tfjs-converter/python/tensorflowjs/quantization.py:93-146, :175-216) for the
synthetic model generators; tests pin it against fixtures produced by importing
the reference module.
"""
from ctypes import c_void_p

import numpy as np

from . import _cabi
from .backend import NP_DTYPES, DataId, TensorInfo, _Record, size_from_shape

DTYPE_VALUE_SIZE_MAP = {"float32": 4, "float16": 2, "int32": 4, "uint16": 2, "uint8": 1,
                        "bool": 1, "complex64": 8}


def dequantize_to_device(backend, q, scale, min_val, shape, dtype):
    """Uploads quantised bytes and dequantises them on the device.
    values[i] = q[i] * scale + min, rounded as io_utils.ts:221-227 (float32) or
    :243-247 (int32, Math.round) does."""
    q = np.ascontiguousarray(q)
    if q.dtype not in (np.uint8, np.uint16):
        raise ValueError("Unsupported quantization dtype %s" % q.dtype)
    if dtype not in ("float32", "int32"):
        raise ValueError("Unsupported quantization type %s for weight type %s." %
                         (q.dtype, dtype))
    n = size_from_shape(shape)
    if q.size != n:
        raise ValueError("dequantize: %d quantised values for shape %s" % (q.size, list(shape)))
    q_id = backend._alloc(q.nbytes)
    out = backend.make_output(shape, dtype)
    try:
        if q.nbytes:
            backend.check(backend.lib.tfjs_cuda_write(backend.ctx, q_id,
                                                      q.ctypes.data_as(c_void_p), q.nbytes))
        backend.check(backend.lib.tfjs_cuda_dequantize(
            backend.ctx, q.dtype.itemsize, _cabi.DTYPES[dtype], q_id, float(scale),
            float(min_val), n, backend.device_id(out.dataId)))
    except Exception:
        backend.disposeData(out.dataId)
        raise
    finally:
        backend.check(backend.lib.tfjs_cuda_free(backend.ctx, q_id))
    return out


def decode_float16_to_device(backend, q, shape):
    """Upload raw float16 bits (uint16) and widen them to float32 on the device
    (io_utils.ts:228-231 with the decoder of :720-741)."""
    q = np.ascontiguousarray(q).view(np.uint16).reshape(-1)
    n = int(q.size)
    out = backend.make_output(shape, "float32")
    if n == 0:
        return out
    qid = backend._alloc(n * 2)
    try:
        backend.check(backend.lib.tfjs_cuda_write(backend.ctx, qid, q.ctypes.data_as(c_void_p),
                                                  n * 2))
        backend.check(backend.lib.tfjs_cuda_decode_float16(backend.ctx, qid, n,
                                                           backend.device_id(out.dataId)))
    except Exception:
        backend.disposeData(out.dataId)
        raise
    finally:
        backend.check(backend.lib.tfjs_cuda_free(backend.ctx, qid))
    return out


def decode_weights(engine, weight_data, specs):
    """name -> Tensor for every manifest entry, in manifest order
    (io_utils.ts:119-135).  `weight_data` is the concatenated little-endian
    buffer; `specs` are WeightsManifestEntry dicts (tfjs-core/src/io/types.ts:76-110)."""
    buf = memoryview(weight_data)
    out = {}
    offset = 0
    for spec in specs:
        name, dtype, shape = spec["name"], spec["dtype"], spec["shape"]
        size = size_from_shape(shape)
        quant = spec.get("quantization")
        if quant is not None:
            qd = quant["dtype"]
            if qd in ("uint8", "uint16"):
                if "min" not in quant or "scale" not in quant:
                    raise ValueError("Weight %s with quantization %s doesn't have "
                                     "corresponding metadata min and scale." % (name, qd))
            elif qd == "float16":
                if dtype != "float32":
                    raise ValueError("Weight %s is quantized with %s which only supports "
                                     "weights of type float32 not %s." % (name, qd, dtype))
            else:
                raise ValueError("Weight %s has unknown quantization dtype %s. Supported "
                                 "quantization dtypes are: 'uint8', 'uint16', and 'float16'."
                                 % (name, qd))
            nbytes = size * DTYPE_VALUE_SIZE_MAP[qd]
            raw = np.frombuffer(buf[offset:offset + nbytes], dtype=np.dtype(qd))
            offset += nbytes
            if qd == "float16":
                engine.ready()
                t = engine.make_tensor_from_info(decode_float16_to_device(engine.backend, raw,
                                                                          shape))
            else:
                if dtype not in ("float32", "int32"):
                    raise ValueError("Unsupported dtype in weight '%s': %s" % (name, dtype))
                engine.ready()
                info = dequantize_to_device(engine.backend, raw, quant["scale"], quant["min"],
                                            shape, dtype)
                t = engine.make_tensor_from_info(info)
        elif dtype == "string":
            raise ValueError("string weights are not supported by the CUDA backend")
        else:
            if dtype not in ("float32", "int32", "bool"):
                raise ValueError("Unsupported dtype in weight '%s': %s" % (name, dtype))
            nbytes = size * DTYPE_VALUE_SIZE_MAP[dtype]
            raw = np.frombuffer(buf[offset:offset + nbytes], dtype=NP_DTYPES[dtype])
            offset += nbytes
            t = engine.make_tensor(raw, shape, dtype)
        out[name] = t
    return out


# ----------------------------------------------------------- native loader --
def _entry(spec):
    """(storage, dtype, elements, stored bytes) of a manifest entry, with the checks of
    decodeWeight (io_utils.ts:196-218, :269-272)."""
    name, dtype, shape = spec["name"], spec["dtype"], spec["shape"]
    n = size_from_shape(shape)
    quant = spec.get("quantization")
    if quant is not None:
        qd = quant["dtype"]
        if qd in ("uint8", "uint16"):
            if "min" not in quant or "scale" not in quant:
                raise ValueError("Weight %s with quantization %s doesn't have "
                                 "corresponding metadata min and scale." % (name, qd))
            if dtype not in ("float32", "int32"):
                raise ValueError("Unsupported dtype in weight '%s': %s" % (name, dtype))
            return (_cabi.STORED_UINT8 if qd == "uint8" else _cabi.STORED_UINT16, dtype, n,
                    n * DTYPE_VALUE_SIZE_MAP[qd])
        if qd == "float16":
            if dtype != "float32":
                raise ValueError("Weight %s is quantized with %s which only supports "
                                 "weights of type float32 not %s." % (name, qd, dtype))
            return _cabi.STORED_FLOAT16, dtype, n, n * 2
        raise ValueError("Weight %s has unknown quantization dtype %s. Supported "
                         "quantization dtypes are: 'uint8', 'uint16', and 'float16'." % (name, qd))
    if dtype == "string":
        raise ValueError("string weights are not supported by the CUDA backend")
    if dtype not in ("float32", "int32", "bool"):
        raise ValueError("Unsupported dtype in weight '%s': %s" % (name, dtype))
    return _cabi.STORED_RAW, dtype, n, n * DTYPE_VALUE_SIZE_MAP[dtype]


class WeightsLoader(object):
    """Drives the library's weight loader (tfjs_cuda_weights_begin / push / push_file /
    end): the bytes of the weight shards, pushed in manifest order in pieces of any size,
    become device tensors without being sliced on the host; quantised and float16-stored
    entries are decoded on the device while the next entry is still being copied.

    Entries no larger than the backend's host-resident limit that are stored in their own
    dtype (shape, axis and permutation constants, small biases) stay on the host, where the
    graph executor reads them without touching the stream: the library passes over their
    bytes and this class collects them from the pieces as they go by."""

    def __init__(self, engine, specs):
        from .backend import HOST_RESIDENT_BYTES
        engine.ready()
        self.engine, self.backend, self.specs = engine, engine.backend, list(specs)
        arr = (_cabi.WeightSpec * max(len(self.specs), 1))()
        self.host = {}          # entry index -> [offset, stored bytes, bytearray]
        offset = 0
        for i, spec in enumerate(self.specs):
            storage, dtype, n, nbytes = _entry(spec)
            q = spec.get("quantization") or {}
            arr[i].n, arr[i].storage, arr[i].dtype = n, storage, _cabi.DTYPES[dtype]
            arr[i].scale, arr[i].min = float(q.get("scale", 1.0)), float(q.get("min", 0.0))
            if storage == _cabi.STORED_RAW and nbytes <= HOST_RESIDENT_BYTES:
                arr[i].skip = 1
                self.host[i] = [offset, nbytes, bytearray(nbytes)]
            offset += nbytes
        self.total = offset
        self.pushed = 0
        handle = _cabi.c_int32()
        self.backend.check(self.backend.lib.tfjs_cuda_weights_begin(
            self.backend.ctx, arr, len(self.specs), _cabi.byref(handle)))
        self.handle = handle.value
        self._starts = sorted((v[0], i) for i, v in self.host.items())

    def _keep_host_parts(self, view, base):
        """Copies the parts of the piece [base, base + len(view)) that belong to
        host-resident entries."""
        end = base + len(view)
        for off, i in self._starts:
            nb = self.host[i][1]
            if off >= end:
                break
            if off + nb <= base or nb == 0:
                continue
            lo, hi = max(off, base), min(off + nb, end)
            self.host[i][2][lo - off:hi - off] = view[lo - base:hi - base]

    def push(self, chunk):
        """One piece of the concatenated weight bytes (bytes, bytearray, memoryview or a
        numpy array)."""
        view = memoryview(chunk).cast("B")
        if len(view) == 0:
            return
        buf = np.frombuffer(view, dtype=np.uint8)
        try:
            self.backend.check(self.backend.lib.tfjs_cuda_weights_push(
                self.backend.ctx, self.handle, buf.ctypes.data_as(c_void_p), len(view)))
        except Exception:
            self.abandon()
            raise
        self._keep_host_parts(view, self.pushed)
        self.pushed += len(view)

    def push_file(self, path):
        """One shard file (an element of weightsManifest[].paths), read by the library."""
        import os
        try:
            self.backend.check(self.backend.lib.tfjs_cuda_weights_push_file(
                self.backend.ctx, self.handle, os.fsencode(path)))
        except Exception:
            self.abandon()
            raise
        base, end = self.pushed, self.pushed + os.path.getsize(path)
        with open(path, "rb") as f:
            for off, i in self._starts:
                nb = self.host[i][1]
                if off >= end or off + nb <= base or nb == 0:
                    continue
                lo, hi = max(off, base), min(off + nb, end)
                f.seek(lo - base)
                self.host[i][2][lo - off:hi - off] = f.read(hi - lo)
        self.pushed = end

    def abandon(self):
        if self.handle:
            handle, self.handle = self.handle, 0
            self.backend.lib.tfjs_cuda_weights_end(self.backend.ctx, handle, None, None)

    def finish(self):
        """name -> Tensor for every entry, in manifest order."""
        ids = (_cabi.c_int32 * max(len(self.specs), 1))()
        handle, self.handle = self.handle, 0
        self.backend.check(self.backend.lib.tfjs_cuda_weights_end(
            self.backend.ctx, handle, ids, None))
        out = {}
        for i, spec in enumerate(self.specs):
            dtype, shape = spec["dtype"], spec["shape"]
            if i in self.host:
                raw = np.frombuffer(bytes(self.host[i][2]), dtype=NP_DTYPES[dtype])
                out[spec["name"]] = self.engine.make_tensor(raw, shape, dtype)
                continue
            nbytes = size_from_shape(shape) * np.dtype(NP_DTYPES[dtype]).itemsize
            data_id = DataId()
            self.backend.data[data_id] = _Record(ids[i], nbytes, dtype, 1, None)
            out[spec["name"]] = self.engine.make_tensor_from_info(TensorInfo(data_id, shape, dtype))
        return out


def load_weights(engine, weight_data, specs):
    """Drop-in for decode_weights through the library's loader: `weight_data` is the
    concatenated buffer, or a list of shard buffers in order (io_utils.ts:119-135)."""
    loader = WeightsLoader(engine, specs)
    shards = weight_data if isinstance(weight_data, (list, tuple)) else [weight_data]
    for shard in shards:
        loader.push(shard)
    return loader.finish()


def load_weights_from_files(engine, paths, specs):
    """The shards of one weights group read from disk by the library, in the order of
    weightsManifest[].paths (weights_loader.ts:38-131 fetches and concatenates them)."""
    loader = WeightsLoader(engine, specs)
    for path in paths:
        loader.push_file(path)
    return loader.finish()


def decode_weights_stream(engine, chunks, specs):
    """decodeWeightsStream (io_utils.ts:316-353): `chunks` is any iterable of byte pieces,
    cut anywhere; each piece is handed to the device loader as it arrives."""
    loader = WeightsLoader(engine, specs)
    try:
        for chunk in chunks:
            loader.push(chunk)
    except Exception:
        loader.abandon()
        raise
    return loader.finish()


# ------------------------------------------------------------ converter side --
def _affine_range(min_val, max_val, qdtype):
    """quantization.py:175-216: nudge the range so that 0.0 maps to an integer."""
    quant_max = np.iinfo(qdtype).max
    scale = (max_val - min_val) / quant_max
    if min_val <= 0 <= max_val:
        nudged_zero = np.round((0 - min_val) / scale)
        nudged_min = -nudged_zero * scale
        nudged_max = quant_max * scale + nudged_min
    else:
        nudged_min, nudged_max = min_val, max_val
    return scale, nudged_min, nudged_max


def quantize_weights(data, qdtype):
    """quantization.py:93-146 for uint8 / uint16: returns (quantised, {min, scale})."""
    qdtype = np.dtype(qdtype).type
    if qdtype not in (np.uint8, np.uint16):
        raise ValueError("Invalid `quantization_dtype`: %r" % qdtype)
    min_val = data.min().astype(np.float64)
    max_val = data.max().astype(np.float64)
    if min_val == max_val:
        return np.zeros_like(data, dtype=qdtype), {"min": min_val, "scale": 1.0}
    scale, min_val, max_val = _affine_range(min_val, max_val, qdtype)
    q = np.round((data.clip(min_val, max_val) - min_val) / scale).astype(qdtype)
    return q, {"min": min_val, "scale": scale}


def encode_weights(named, quantize=None):
    """Concatenated weight bytes plus manifest entries, in order
    (tfjs-core/src/io/io_utils.ts:52-101 / write_weights.py).  `quantize` is None,
    'uint8' or 'uint16' and applies to float32 tensors with more than one element."""
    specs, chunks = [], []
    for name, arr in named:
        arr = np.asarray(arr)
        if arr.dtype == np.bool_:
            dtype, raw = "bool", arr.astype(np.uint8)
        elif np.issubdtype(arr.dtype, np.integer):
            dtype, raw = "int32", arr.astype(np.int32)
        else:
            dtype, raw = "float32", arr.astype(np.float32)
        spec = {"name": name, "shape": [int(s) for s in arr.shape], "dtype": dtype}
        if quantize and dtype == "float32" and arr.size > 1 and arr.ndim > 1:
            q, meta = quantize_weights(raw, np.dtype(quantize))
            spec["quantization"] = {"dtype": quantize, "min": float(meta["min"]),
                                    "scale": float(meta["scale"])}
            raw = q
        specs.append(spec)
        chunks.append(np.ascontiguousarray(raw).tobytes())
    return b"".join(chunks), specs
