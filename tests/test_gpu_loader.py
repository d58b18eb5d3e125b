"""The library's weight loader against the per-tensor decode path (B200 only).

tfjs_cuda_weights_begin / push / push_file / end take the weight bytes in pieces cut
anywhere, stage them through pinned memory and decode quantised entries on the device.
Every tensor must carry the bits io.decode_weights produces (which the oracle tests pin to
the reference's decodeWeights), whatever the piece sizes, from memory, from shard files and
as a stream; wrong byte counts must fail cleanly and leave nothing behind.
"""
import json
import os

import numpy as np
import pytest

from tfjs_b200 import io, model_zoo
from tfjs_b200.graph_model import GraphModel

pytestmark = pytest.mark.gpu


def _mixed_manifest(seed=4):
    """Entries of every storage kind, sizes from empty to larger than a staging slot."""
    r = np.random.default_rng(seed)
    named, specs, chunks = [], [], []

    def add(name, arr, dtype, quant=None):
        spec = {"name": name, "shape": list(arr.shape), "dtype": dtype}
        if quant:
            spec["quantization"] = quant
        specs.append(spec)
        chunks.append(np.ascontiguousarray(arr).tobytes())

    add("f32_big", r.standard_normal((5, 1024, 1031)).astype(np.float32), "float32")   # 21 MB
    add("axis", np.array([1, 2], np.int32), "int32")                                  # host-resident
    add("empty", np.zeros((0, 3), np.float32), "float32")
    add("q8", r.integers(0, 256, (3, 3, 64, 67)).astype(np.uint8), "float32",
        {"dtype": "uint8", "scale": 0.0123, "min": -1.57})
    add("scalar", np.array(2.5, np.float32), "float32")
    add("q16", r.integers(0, 65536, (1000, 77)).astype(np.uint16), "float32",
        {"dtype": "uint16", "scale": 3.1e-5, "min": -1.0})
    add("q8_int", r.integers(0, 256, (4099,)).astype(np.uint8), "int32",
        {"dtype": "uint8", "scale": 0.37, "min": -40.25})
    half = r.standard_normal(70001).astype(np.float16)
    half[:6] = np.array([np.nan, np.inf, -np.inf, 6e-8, -0.0, 65504.0], np.float16)
    add("f16", half.view(np.uint16), "float32", {"dtype": "float16"})
    add("flags", (r.random(5000) < 0.5).astype(np.uint8), "bool")
    add("ids", r.integers(-5, 5, (2048, 3)).astype(np.int32), "int32")
    add("q16_int", r.integers(0, 65536, (513,)).astype(np.uint16), "int32",
        {"dtype": "uint16", "scale": 0.0417, "min": -900.5})
    return specs, b"".join(chunks)


def _same(a, b):
    assert list(a) == list(b)
    for name in a:
        ta, tb = a[name], b[name]
        assert ta.shape == tb.shape and ta.dtype == tb.dtype, name
        va, vb = ta.dataSync(), tb.dataSync()
        if ta.dtype == "float32":
            va, vb = va.view(np.uint32), vb.view(np.uint32)
        assert np.array_equal(va, vb), name


def _dispose(*maps):
    for m in maps:
        for t in m.values():
            t.dispose()


def _pieces(data, sizes):
    """Cuts data into pieces of the given sizes, cycling through them."""
    out, off, k = [], 0, 0
    while off < len(data):
        n = sizes[k % len(sizes)]
        out.append(data[off:off + n])
        off += n
        k += 1
    return out


@pytest.mark.parametrize("sizes", [[1 << 40], [1, 7, 4097, 1 << 20], [(9 << 20) + 5], [123457]])
def test_loader_matches_per_tensor_decode_for_any_piece_size(cuda_engine, sizes):
    specs, data = _mixed_manifest()
    want = io.decode_weights(cuda_engine, data, specs)
    got = io.decode_weights_stream(cuda_engine, iter(_pieces(data, sizes)), specs)
    _same(got, want)
    # the small entries stayed on the host, as with the per-tensor path
    assert cuda_engine.backend.host_values(got["axis"].dataId) is not None
    _dispose(got, want)


def test_resnet50_uint8_artifacts_from_ragged_shards(cuda_engine):
    model_json, weights = model_zoo.resnet50(1, size=32)
    specs = model_json["weightsManifest"][0]["weights"]
    assert sum("quantization" in s for s in specs) > 50
    want = io.decode_weights(cuda_engine, weights, specs)
    cut = [0, 4 * 1000 * 1000 + 3, 11 * 1000 * 1000 + 1, len(weights)]
    shards = [weights[a:b] for a, b in zip(cut[:-1], cut[1:])]
    got = io.load_weights(cuda_engine, shards, specs)
    _same(got, want)
    _dispose(got, want)


def test_graph_model_loads_shard_files_by_path(cuda_engine, tmp_path):
    model_json, weights = model_zoo.mobilenet_v2(2, size=96)
    cut = [0, 1234567, 5000001, len(weights)]
    names = ["group1-shard%dof3.bin" % (i + 1) for i in range(3)]
    for name, a, b in zip(names, cut[:-1], cut[1:]):
        (tmp_path / name).write_bytes(weights[a:b])
    on_disk = dict(model_json)
    on_disk["weightsManifest"] = [dict(model_json["weightsManifest"][0], paths=names)]
    (tmp_path / "model.json").write_text(json.dumps(on_disk))
    from_files = GraphModel.load(str(tmp_path / "model.json"), cuda_engine)
    in_memory = GraphModel(model_json, weights, cuda_engine, decode_weights=io.decode_weights)
    _same(from_files.weights, in_memory.weights)
    x = cuda_engine.make_tensor(np.random.default_rng(1).uniform(-1, 1, (2, 96, 96, 3))
                                .astype(np.float32))
    a, b = from_files.execute(x), in_memory.execute(x)
    assert np.array_equal(a.dataSync().view(np.uint32), b.dataSync().view(np.uint32))
    for t in (x, a, b):
        t.dispose()
    from_files.dispose()
    in_memory.dispose()


def test_wrong_byte_counts_fail_and_leave_nothing_behind(cuda_engine, tmp_path):
    from tfjs_b200.backend import CudaError
    specs, data = _mixed_manifest()
    be = cuda_engine.backend
    before = (be.numDataIds(), be.memory()["numDeviceBuffers"])
    with pytest.raises(CudaError, match="were pushed"):
        io.load_weights(cuda_engine, data[:-5], specs)
    with pytest.raises(CudaError, match="beyond what the manifest entries hold"):
        io.load_weights(cuda_engine, data + b"123", specs)
    with pytest.raises(CudaError, match="No such file"):
        io.load_weights_from_files(cuda_engine, [str(tmp_path / "missing.bin")], specs)
    bad = [dict(specs[3], quantization={"dtype": "uint4", "scale": 1, "min": 0})]
    with pytest.raises(ValueError, match="unknown quantization dtype"):
        io.load_weights(cuda_engine, b"", bad)
    assert (be.numDataIds(), be.memory()["numDeviceBuffers"]) == before
    # the context still loads
    got = io.load_weights(cuda_engine, data, specs)
    want = io.decode_weights(cuda_engine, data, specs)
    _same(got, want)
    _dispose(got, want)
