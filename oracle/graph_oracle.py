"""TEST INFRASTRUCTURE ONLY -- runs a graph-model artifact (model.json + weight
bytes) on the CPU oracle and returns every node's output.

It restates what the reference does for these artifacts: decodeWeights
(tfjs-core/src/io/io_utils.ts:119-135, :185-292) followed by the converter's
per-op executors (tfjs-converter/src/operations/executors/*.ts) calling
tfjs-backend-cpu kernels.  Independent of the product's graph runner.
"""
import base64

import numpy as np

from . import oracle as orc

_DT = {"float32": np.float32, "int32": np.int32, "bool": np.uint8}
_QSIZE = {"uint8": 1, "uint16": 2, "float16": 2}


def decode_weights(weight_data, specs):
    out, off = {}, 0
    buf = memoryview(weight_data)
    for s in specs:
        n = int(np.prod(s["shape"], dtype=np.int64))
        q = s.get("quantization")
        if q:
            nb = n * _QSIZE[q["dtype"]]
            raw = np.frombuffer(buf[off:off + nb], dtype=np.dtype(q["dtype"]))
            off += nb
            if q["dtype"] == "float16":
                val = raw.astype(np.float32)
            else:
                val = orc.dequantize(raw, q["scale"], q["min"], s["dtype"])
        else:
            nb = n * np.dtype(_DT[s["dtype"]]).itemsize
            val = np.frombuffer(buf[off:off + nb], dtype=_DT[s["dtype"]]).copy()
            off += nb
        out[s["name"]] = val.reshape(s["shape"])
    return out


def _s(attr, name, default=None):
    a = attr.get(name)
    if not a or "s" not in a:
        return default
    return base64.b64decode(a["s"]).decode().lower()


def _ints(attr, name, default=None):
    a = attr.get(name)
    if not a or "list" not in a or not a["list"].get("i"):
        return default
    return [int(v) for v in a["list"]["i"]]


def _b(attr, name):
    a = attr.get(name)
    return bool(a and a.get("b"))


def _fused(attr):
    ops = [base64.b64decode(s).decode().lower() for s in attr["fused_ops"]["list"]["s"]]
    assert ops[0] == "biasadd"
    return ops[1] if len(ops) > 1 else "linear"


def run(model_json, weight_data, inputs, stop_after=None):
    """Returns {node name: numpy output} for every executed node."""
    specs = []
    for group in model_json["weightsManifest"]:
        specs.extend(group["weights"])
    vals = decode_weights(weight_data, specs)
    vals.update(inputs)
    for node in model_json["modelTopology"]["node"]:
        op, name, attr = node["op"], node["name"], node.get("attr", {})
        if op in ("Const", "Placeholder"):
            continue
        x = [vals[i.split(":")[0]] for i in node.get("input", [])]
        if op in ("_FusedConv2D", "FusedDepthwiseConv2dNative"):
            st, dl = _ints(attr, "strides"), _ints(attr, "dilations", [1, 1, 1, 1])
            fn = orc.fused_conv2d if op == "_FusedConv2D" else orc.fused_depthwise_conv2d
            y = fn(x[0], x[1], [st[1], st[2]], _s(attr, "padding"), [dl[1], dl[2]], None,
                   bias=x[2], activation=_fused(attr), leakyrelu_alpha=0.2)
        elif op == "_FusedMatMul":
            y = orc.fused_matmul(x[0], x[1], _b(attr, "transpose_a"), _b(attr, "transpose_b"),
                                 bias=x[2], activation=_fused(attr), leakyrelu_alpha=0.2)
        elif op == "BatchMatMulV2":
            y = orc.batch_matmul(x[0], x[1], _b(attr, "adj_x"), _b(attr, "adj_y"))
        elif op == "MaxPool":
            k, st = _ints(attr, "ksize"), _ints(attr, "strides")
            y = orc.pool2d(x[0], "max", [k[1], k[2]], [st[1], st[2]], _s(attr, "padding"))
        elif op == "Mean":
            y = orc.reduce("mean", x[0], [int(v) for v in x[1].reshape(-1)], _b(attr, "keep_dims"))
        elif op in ("AddV2", "Sub", "Mul", "SquaredDifference", "RealDiv"):
            y = orc.binary({"AddV2": "add", "Sub": "sub", "Mul": "mul", "RealDiv": "div",
                            "SquaredDifference": "squared_difference"}[op], x[0], x[1])
        elif op in ("Relu", "Relu6", "Rsqrt", "Erf", "Sqrt", "Tanh", "Exp"):
            y = orc.unary(op.lower(), x[0])
        elif op == "Softmax":
            y = orc.softmax(x[0])
        elif op == "GatherV2":
            y = orc.gather(x[0], x[1], int(x[2].reshape(-1)[0]))
        elif op == "Reshape":
            y = np.ascontiguousarray(x[0]).reshape([int(v) for v in x[1].reshape(-1)])
        elif op == "Transpose":
            y = orc.transpose(x[0], [int(v) for v in x[1].reshape(-1)])
        else:
            raise NotImplementedError(op)
        vals[name] = y
        if stop_after == name:
            break
    return vals
