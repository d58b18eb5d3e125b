"""Generates quantisation fixtures by importing the reference's own module.

    python tests/golden/make_quant_goldens.py <tfjs checkout> tests/golden/quant_goldens.npz

tfjs-converter/python/tensorflowjs/quantization.py needs only numpy, so it is
loaded straight from the reference checkout (the `tensorflowjs` package itself
cannot be imported: its __init__ pulls in TensorFlow).  For seeded float32
tensors the fixture stores what `quantize_weights` returned (quantised values,
min, scale) and what `dequantize_weights` reconstructs; tests check the repo's
restatements against them.  The io_utils dequantisation known answers
(tfjs-core/src/io/io_utils_test.ts:546-601: min -1, scale 0.1, values
[0, 48, 255] -> float32 [-1, 3.8, 24.5], int32 [-1, 4, 25]) are stored as well.
"""
import importlib.util
import os
import sys

import numpy as np


def main(ref_root, out_path):
    path = os.path.join(ref_root, "tfjs-converter/python/tensorflowjs/quantization.py")
    spec = importlib.util.spec_from_file_location("ref_quantization", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    out = {}
    r = np.random.default_rng(1234)
    tensors = {
        "normal": (r.standard_normal((37, 19)) * 0.07).astype(np.float32),
        "positive": (np.abs(r.standard_normal(500)) + 0.5).astype(np.float32),
        "negative": (-np.abs(r.standard_normal(300)) - 0.25).astype(np.float32),
        "wide": (r.standard_normal((3, 3, 16, 8)) * 3.0).astype(np.float32),
        "constant": np.full((4, 4), 0.75, np.float32),
        "two_values": np.array([-1.0, 2.0, 2.0, -1.0], np.float32),
    }
    names = []
    for name, data in tensors.items():
        for qname, qdt in (("uint8", np.uint8), ("uint16", np.uint16)):
            q, meta = mod.quantize_weights(data, qdt)
            deq = mod.dequantize_weights(q, meta, np.float32)
            key = "%s_%s" % (name, qname)
            names.append(key)
            out[key + "_data"] = data
            out[key + "_q"] = q
            out[key + "_min"] = np.float64(meta["min"])
            out[key + "_scale"] = np.float64(meta["scale"])
            out[key + "_deq"] = deq
    out["names"] = np.array(names)
    out["io_utils_q"] = np.array([0, 48, 255], np.uint8)
    out["io_utils_min"] = np.float64(-1)
    out["io_utils_scale"] = np.float64(0.1)
    out["io_utils_f32"] = np.array([-1, 3.8, 24.5], np.float32)
    out["io_utils_i32"] = np.array([-1, 4, 25], np.int32)
    np.savez_compressed(out_path, **out)
    print("wrote %d quantisation fixtures to %s" % (len(names), out_path))


if __name__ == "__main__":
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    if len(sys.argv) < 2:
        sys.exit("usage: %s <path to a tensorflow/tfjs checkout> [output file]" % sys.argv[0])
    main(sys.argv[1],
         sys.argv[2] if len(sys.argv) > 2 else os.path.join(root, "tests/golden/quant_goldens.npz"))
