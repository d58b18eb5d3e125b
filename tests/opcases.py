"""Runs one op case {op, inputs, attrs} on the CPU oracle or on the CUDA backend.

The same case format is used by the golden vectors extracted from the
reference's tests and by the seeded random parity tests, so both the oracle and
the CUDA path are checked with identical inputs.
"""
import numpy as np

from oracle import oracle as orc

UNARY = ("relu", "relu6", "elu", "sigmoid", "exp", "sqrt", "rsqrt", "square", "tanh", "neg",
         "erf", "abs", "log")
BINARY = {"add": "add", "sub": "sub", "mul": "mul", "div": "div", "maximum": "maximum",
          "minimum": "minimum", "pow": "pow", "squared_difference": "squared_difference"}


def _conv_kw(a):
    return dict(strides=a.get("strides", 1), pad=a.get("pad", "valid"),
                dilations=a.get("dilations", 1) or 1,
                rounding_mode=a.get("dimRoundingMode"))


def _fused_kw(i, a):
    return dict(bias=i.get("bias"), activation=a.get("activation", "linear") or "linear",
                prelu_weights=i.get("preluActivationWeights"),
                leakyrelu_alpha=a.get("leakyreluAlpha", 0.2))


def run_oracle(case):
    op, i, a = case["op"], case["inputs"], case.get("attrs", {})
    if a.get("dataFormat", "NHWC") == "NCHW":
        raise NotImplementedError("NCHW")
    if op == "fused_conv2d":
        return orc.fused_conv2d(i["x"], i["filter"], **_conv_kw(a), **_fused_kw(i, a))
    if op == "conv2d":
        return orc.conv2d(i["x"], i["filter"], **_conv_kw(a))
    if op == "fused_depthwise_conv2d":
        return orc.fused_depthwise_conv2d(i["x"], i["filter"], **_conv_kw(a), **_fused_kw(i, a))
    if op == "depthwise_conv2d":
        return orc.depthwise_conv2d(i["x"], i["filter"], **_conv_kw(a))
    if op == "mat_mul":
        return orc.batch_matmul(i["a"], i["b"], a.get("transposeA", False),
                                a.get("transposeB", False))
    if op == "fused_mat_mul":
        return orc.fused_matmul(i["a"], i["b"], a.get("transposeA", False),
                                a.get("transposeB", False), **_fused_kw(i, a))
    if op in ("max_pool", "avg_pool"):
        return orc.pool2d(i["x"], "max" if op == "max_pool" else "avg", a["filterSize"],
                          a["strides"], a["pad"], a.get("dimRoundingMode"))
    if op in UNARY:
        return orc.unary(op, i["x"])
    if op == "leaky_relu":
        return orc.unary("leakyrelu", i["x"], a.get("alpha", 0.2))
    if op == "clip_by_value":
        return orc.unary("clip", i["x"], a["lo"], a["hi"])
    if op in BINARY:
        return orc.binary(BINARY[op], i["a"], i["b"])
    if op == "prelu":
        return orc.binary("prelu", i["x"], i["alpha"])
    if op == "softmax":
        return orc.softmax(i["logits"], a.get("dim", -1))
    if op in ("sum", "mean", "max"):
        return orc.reduce(op, i["x"], a.get("axis"), a.get("keepDims", False))
    if op == "arg_max":
        return orc.argmax(i["x"], a.get("axis", 0))
    if op == "transpose":
        x = np.asarray(i["x"])
        return orc.transpose(x, a.get("perm") or list(range(x.ndim))[::-1])
    if op == "gather":
        return orc.gather(i["x"], i["indices"], a.get("axis", 0), a.get("batchDims", 0))
    if op == "cast":
        return orc.cast(i["x"], a["dtype"])
    if op == "batch_norm":
        return orc.batch_norm(i["x"], i["mean"], i["variance"], i.get("offset"),
                              i.get("scale"), a.get("varianceEpsilon"))
    if op == "concat":
        return np.concatenate([np.asarray(t) for t in i["tensors"]], a.get("axis", 0))
    if op == "slice":
        x = np.asarray(i["x"])
        begin, size = a["begin"], a.get("size")
        begin = list(begin) if isinstance(begin, (list, tuple)) else [begin]
        begin += [0] * (x.ndim - len(begin))
        if size is None:
            size = [-1] * x.ndim
        size = list(size) if isinstance(size, (list, tuple)) else [size]
        size += [-1] * (x.ndim - len(size))
        sl = tuple(slice(b, None if s < 0 else b + s) for b, s in zip(begin, size))
        return x[sl].copy()
    if op == "pad":
        return np.pad(np.asarray(i["x"]), a["paddings"], constant_values=a.get("constantValue", 0))
    if op == "tile":
        return np.tile(np.asarray(i["x"]), a["reps"])
    if op == "stack":
        return np.stack([np.asarray(t) for t in i["tensors"]], a.get("axis", 0))
    if op == "expand_dims":
        return np.expand_dims(np.asarray(i["x"]), a.get("axis", 0))
    raise NotImplementedError(op)


def run_cuda(case):
    """Runs the case through the 'cuda' backend ops; returns a numpy array."""
    from tfjs_b200 import ops
    op, i, a = case["op"], case["inputs"], case.get("attrs", {})
    made = []

    def T(v, dtype=None):
        if v is None:
            return None
        arr = np.asarray(v)
        if dtype is None:
            dtype = ("bool" if arr.dtype == np.bool_ else
                     "int32" if np.issubdtype(arr.dtype, np.integer) else "float32")
        t = ops.tensor(arr, list(arr.shape), dtype)
        made.append(t)
        return t

    def D(v):
        """A tensor produced by a device kernel (not a host write), so that paths
        reserved for activations, not weights, are taken."""
        t = T(v)
        one = T(np.ones((), np.float32))
        out = ops.mul(t, one)
        made.append(out)
        return out

    dev_in = set(case.get("device_inputs", ()))
    try:
        if op in ("fused_conv2d", "fused_depthwise_conv2d"):
            fn = ops.fused_conv2d if op == "fused_conv2d" else ops.fused_depthwise_conv2d
            out = fn(T(i["x"]), T(i["filter"]), a.get("strides", 1), a.get("pad", "valid"),
                     a.get("dataFormat", "NHWC"), a.get("dilations", [1, 1]) or [1, 1],
                     a.get("dimRoundingMode"), T(i.get("bias")),
                     a.get("activation", "linear") or "linear",
                     T(i.get("preluActivationWeights")), a.get("leakyreluAlpha"))
        elif op in ("conv2d", "depthwise_conv2d"):
            fn = ops.conv2d if op == "conv2d" else ops.depthwise_conv2d
            out = fn(T(i["x"]), T(i["filter"]), a.get("strides", 1), a.get("pad", "valid"),
                     a.get("dataFormat", "NHWC"), a.get("dilations", [1, 1]) or [1, 1],
                     a.get("dimRoundingMode"))
        elif op == "mat_mul":
            out = ops.mat_mul(T(i["a"]), (D if "b" in dev_in else T)(i["b"]),
                              a.get("transposeA", False), a.get("transposeB", False))
        elif op == "fused_mat_mul":
            out = ops.fused_mat_mul(T(i["a"]), (D if "b" in dev_in else T)(i["b"]),
                                    a.get("transposeA", False),
                                    a.get("transposeB", False), T(i.get("bias")),
                                    a.get("activation", "linear") or "linear",
                                    T(i.get("preluActivationWeights")),
                                    a.get("leakyreluAlpha", 0.2))
        elif op in ("max_pool", "avg_pool"):
            fn = ops.max_pool if op == "max_pool" else ops.avg_pool
            out = fn(T(i["x"]), a["filterSize"], a["strides"], a["pad"], a.get("dimRoundingMode"))
        elif op in UNARY:
            out = getattr(ops, op)(T(i["x"]))
        elif op == "leaky_relu":
            out = ops.leaky_relu(T(i["x"]), a.get("alpha", 0.2))
        elif op == "clip_by_value":
            out = ops.clip_by_value(T(i["x"]), a["lo"], a["hi"])
        elif op in BINARY:
            out = getattr(ops, op)(T(i["a"]), T(i["b"]))
        elif op == "prelu":
            out = ops.prelu(T(i["x"]), T(i["alpha"]))
        elif op == "softmax":
            out = ops.softmax(T(i["logits"]), a.get("dim", -1))
        elif op in ("sum", "mean", "max"):
            out = getattr(ops, op)(T(i["x"]), a.get("axis"), a.get("keepDims", False))
        elif op == "arg_max":
            out = ops.arg_max(T(i["x"]), a.get("axis", 0))
        elif op == "transpose":
            out = ops.transpose(T(i["x"]), a.get("perm"))
        elif op == "gather":
            out = ops.gather(T(i["x"]), T(i["indices"], "int32"), a.get("axis", 0),
                             a.get("batchDims", 0))
        elif op == "cast":
            out = ops.cast(T(i["x"]), a["dtype"])
        elif op == "batch_norm":
            out = ops.batch_norm(T(i["x"]), T(i["mean"]), T(i["variance"]), T(i.get("offset")),
                                 T(i.get("scale")), a.get("varianceEpsilon"))
        elif op == "concat":
            out = ops.concat([T(t) for t in i["tensors"]], a.get("axis", 0))
        elif op == "slice":
            out = ops.slice(T(i["x"]), a["begin"], a.get("size"))
        elif op == "pad":
            out = ops.pad(T(i["x"]), a["paddings"], a.get("constantValue", 0))
        elif op == "tile":
            out = ops.tile(T(i["x"]), a["reps"])
        elif op == "stack":
            out = ops.stack([T(t) for t in i["tensors"]], a.get("axis", 0))
        elif op == "expand_dims":
            out = ops.expand_dims(T(i["x"]), a.get("axis", 0))
        else:
            raise NotImplementedError(op)
        res = out.arraySync()
        out.dispose()
        return res
    finally:
        for t in made:
            t.dispose()
