"""GraphModel / GraphExecutor for tfjs graph-model artifacts.

Consumes the converter's `model.json` + weight bytes
(tfjs-core/src/io/types.ts:49-110) and runs the node list through the 'cuda'
backend's kernels by way of the same ops the converter's executors call.  The
structure follows the reference: GraphModel.loadSync -> decodeWeights ->
executor (tfjs-converter/src/executor/graph_model.ts:176-234); execute ->
compile once per (inputs, outputs) -> node loop that stores outputs and
disposes each intermediate right after its last consumer has been enqueued
(graph_executor.ts:231-318, :382-409; liveness model_analysis.ts:275-335);
per-op mapping as in operations/executors/*.ts, with attribute decoding as
operation_mapper.ts:437-461 (strings are base64, ints are JSON strings).

In a Node deployment the unmodified tfjs-converter plays this role; this module
drives the same kernels from Python and is what the benchmark times.
"""
import base64
import json
import os

import numpy as np

from . import io, ops
from .engine import ENGINE, Tensor

DT_MAP = {"DT_FLOAT": "float32", "DT_INT32": "int32", "DT_BOOL": "bool", "DT_INT64": "int32",
          1: "float32", 3: "int32", 9: "int32", 10: "bool"}


# ---------------------------------------------------------- attribute values --
def _b64(s):
    try:
        return base64.b64decode(s).decode("utf-8")
    except Exception:
        return s


def attr_string(attrs, name, default=None, keep_case=False):
    """operation_mapper.ts:437-445: base64-decoded and lower-cased."""
    a = attrs.get(name)
    if a is None or "s" not in a:
        return default
    v = _b64(a["s"])
    return v if keep_case else v.lower()


def attr_number(attrs, name, default=None):
    a = attrs.get(name)
    if a is None:
        return default
    if "i" in a:
        return int(a["i"])
    if "f" in a:
        return float(a["f"])
    return default


def attr_bool(attrs, name, default=False):
    a = attrs.get(name)
    if a is None or "b" not in a:
        return default
    return bool(a["b"])


def attr_number_list(attrs, name, default=None):
    a = attrs.get(name)
    if a is None or "list" not in a:
        return default
    lst = a["list"]
    if lst.get("i"):
        return [int(v) for v in lst["i"]]
    if lst.get("f"):
        return [float(v) for v in lst["f"]]
    return default if default is not None else []


def attr_string_list(attrs, name, default=None):
    a = attrs.get(name)
    if a is None or "list" not in a or not a["list"].get("s"):
        return default if default is not None else []
    return [_b64(s).lower() for s in a["list"]["s"]]


def attr_dtype(attrs, name, default=None):
    a = attrs.get(name)
    if a is None or "type" not in a:
        return default
    t = a["type"]
    if t not in DT_MAP:
        raise ValueError("Unsupported dtype %s" % t)
    return DT_MAP[t]


def attr_shape(attrs, name):
    a = attrs.get(name)
    if a is None or "shape" not in a:
        return None
    if a["shape"].get("unknownRank"):
        return None
    return [int(d.get("size", -1)) for d in a["shape"].get("dim", [])]


class Node(object):
    __slots__ = ("name", "op", "inputs", "attrs", "children")

    def __init__(self, d):
        self.name = d["name"]
        self.op = d["op"]
        # control-dependency inputs ("^name") carry no tensor
        self.inputs = [i for i in d.get("input", []) if not i.startswith("^")]
        self.attrs = d.get("attr", {})
        self.children = []


def parse_node_name(name):
    """executors/utils.ts:120-132: 'node:1' -> ('node', 1)."""
    parts = name.split(":")
    if len(parts) == 1:
        return name, 0
    return parts[0], int(parts[-1])


# ------------------------------------------------------------- op executors --
def _vals(t):
    """Small parameter tensors are read on the host (executors/utils.ts:55)."""
    return t.dataSync()


def _pad_param(node):
    pad = attr_string(node.attrs, "padding", "valid")
    if pad == "explicit":
        flat = attr_number_list(node.attrs, "explicit_paddings", [0] * 8)
        return [[flat[2 * i], flat[2 * i + 1]] for i in range(4)]
    return pad


def _fused_params(node, inputs):
    fused = attr_string_list(node.attrs, "fused_ops")
    extra = fused[0] if len(fused) > 0 else None
    activation = fused[1] if len(fused) > 1 else None
    is_bias, is_prelu = extra == "biasadd", activation == "prelu"
    num_args = attr_number(node.attrs, "num_args", 0)
    if is_bias:
        if is_prelu and num_args != 2:
            raise ValueError("FusedConv2d and DepthwiseConv2d with BiasAdd and Prelu must have "
                             "two extra arguments: bias and alpha.")
        if not is_prelu and num_args != 1:
            raise ValueError("FusedConv2d and DepthwiseConv2d with BiasAdd must have one extra "
                             "argument: bias.")
    if extra == "fusedbatchnorm":
        raise ValueError("FusedConv2d and DepthwiseConv2d with FusedBatchNorm is not supported")
    args = list(inputs[2:])
    bias = args[0] if len(args) > 0 else None
    prelu = args[1] if len(args) > 1 else None
    if not is_bias:
        prelu, bias = bias, None
    return bias, prelu, activation or "linear", attr_number(node.attrs, "leakyrelu_alpha", 0.2)


def _exec_conv(node, inp):
    strides = attr_number_list(node.attrs, "strides", [1, 1, 1, 1])
    dil = attr_number_list(node.attrs, "dilations", [1, 1, 1, 1])
    fmt = attr_string(node.attrs, "data_format", "nhwc").upper()
    pad = _pad_param(node)
    if node.op in ("Conv2D", "DepthwiseConv2dNative", "DepthwiseConv2d"):
        fn = ops.conv2d if node.op == "Conv2D" else ops.depthwise_conv2d
        return fn(inp[0], inp[1], [strides[1], strides[2]], pad, fmt, [dil[1], dil[2]])
    bias, prelu, act, alpha = _fused_params(node, inp)
    fn = ops.fused_conv2d if node.op == "_FusedConv2D" else ops.fused_depthwise_conv2d
    return fn(inp[0], inp[1], [strides[1], strides[2]], pad, fmt, [dil[1], dil[2]], None, bias,
              act, prelu, alpha)


def _exec_matmul(node, inp):
    if node.op == "_FusedMatMul":
        bias, prelu, act, alpha = _fused_params(node, inp)
        return ops.fused_mat_mul(inp[0], inp[1], attr_bool(node.attrs, "transpose_a"),
                                 attr_bool(node.attrs, "transpose_b"), bias, act, prelu, alpha)
    if node.op == "MatMul":
        return ops.mat_mul(inp[0], inp[1], attr_bool(node.attrs, "transpose_a"),
                           attr_bool(node.attrs, "transpose_b"))
    return ops.mat_mul(inp[0], inp[1], attr_bool(node.attrs, "adj_x"),
                       attr_bool(node.attrs, "adj_y"))


def _exec_pool(node, inp):
    k = attr_number_list(node.attrs, "ksize", [1, 1, 1, 1])
    s = attr_number_list(node.attrs, "strides", [1, 1, 1, 1])
    fn = ops.max_pool if node.op == "MaxPool" else ops.avg_pool
    return fn(inp[0], [k[1], k[2]], [s[1], s[2]], _pad_param(node))


def _exec_reduce(node, inp):
    axis = [int(v) for v in _vals(inp[1])]
    keep = attr_bool(node.attrs, "keep_dims")
    return {"Mean": ops.mean, "Sum": ops.sum, "Max": ops.max}[node.op](inp[0], axis, keep)


_BINARY = {"Add": ops.add, "AddV2": ops.add, "BiasAdd": ops.add, "Sub": ops.sub, "Mul": ops.mul,
           "RealDiv": ops.div, "Div": ops.div, "Maximum": ops.maximum, "Minimum": ops.minimum,
           "Pow": ops.pow, "SquaredDifference": ops.squared_difference}
_UNARY = {"Relu": ops.relu, "Relu6": ops.relu6, "Elu": ops.elu, "Sigmoid": ops.sigmoid,
          "Exp": ops.exp, "Sqrt": ops.sqrt, "Rsqrt": ops.rsqrt, "Square": ops.square,
          "Tanh": ops.tanh, "Neg": ops.neg, "Erf": ops.erf, "Abs": ops.abs, "Log": ops.log}


def execute_op(node, inp):
    """operations/operation_executor.ts:55-124 for the ops of the three models."""
    op = node.op
    if op in ("_FusedConv2D", "FusedDepthwiseConv2dNative", "Conv2D", "DepthwiseConv2dNative",
              "DepthwiseConv2d"):
        return _exec_conv(node, inp)
    if op in ("_FusedMatMul", "MatMul", "BatchMatMul", "BatchMatMulV2"):
        return _exec_matmul(node, inp)
    if op in ("MaxPool", "AvgPool"):
        return _exec_pool(node, inp)
    if op in ("Mean", "Sum", "Max"):
        return _exec_reduce(node, inp)
    if op in _BINARY:
        return _BINARY[op](inp[0], inp[1])
    if op in _UNARY:
        return _UNARY[op](inp[0])
    if op == "LeakyRelu":
        return ops.leaky_relu(inp[0], attr_number(node.attrs, "alpha", 0.2))
    if op == "Prelu":
        return ops.prelu(inp[0], inp[1])
    if op == "ClipByValue":
        return ops.clip_by_value(inp[0], float(_vals(inp[1])[0]), float(_vals(inp[2])[0]))
    if op == "Softmax":
        return ops.softmax(inp[0])
    if op == "ArgMax":
        return ops.arg_max(inp[0], int(_vals(inp[1])[0]))
    if op == "GatherV2":
        return ops.gather(inp[0], inp[1] if inp[1].dtype == "int32" else ops.cast(inp[1], "int32"),
                          int(_vals(inp[2])[0]), attr_number(node.attrs, "batch_dims", 0))
    if op == "Reshape":
        return ops.reshape(inp[0], [int(v) for v in _vals(inp[1])])
    if op == "Transpose":
        return ops.transpose(inp[0], [int(v) for v in _vals(inp[1])])
    if op == "ExpandDims":
        return ops.expand_dims(inp[0], int(_vals(inp[1])[0]))
    if op == "Squeeze":
        dims = attr_number_list(node.attrs, "squeeze_dims", [])
        shape = inp[0].shape
        dims = [d % len(shape) for d in dims] if dims else [i for i, s in enumerate(shape) if s == 1]
        return ops.reshape(inp[0], [s for i, s in enumerate(shape) if i not in dims])
    if op == "ConcatV2":
        return ops.concat(inp[:-1], int(_vals(inp[-1])[0]))
    if op in ("Pad", "PadV2"):
        p = _vals(inp[1]).reshape(-1, 2)
        const = float(_vals(inp[2])[0]) if op == "PadV2" and len(inp) > 2 else \
            attr_number(node.attrs, "constant_value", 0)
        return ops.pad(inp[0], [[int(a), int(b)] for a, b in p], const)
    if op == "Slice":
        return ops.slice(inp[0], [int(v) for v in _vals(inp[1])], [int(v) for v in _vals(inp[2])])
    if op == "Tile":
        return ops.tile(inp[0], [int(v) for v in _vals(inp[1])])
    if op == "Pack":
        return ops.stack(inp, attr_number(node.attrs, "axis", 0))
    if op == "Cast":
        return ops.cast(inp[0], attr_dtype(node.attrs, "DstT", "float32"))
    if op in ("Identity", "StopGradient", "PlaceholderWithDefault"):
        return ops.identity(inp[0])
    if op == "_FusedLayerNorm":
        return _exec_layer_norm(node, inp)
    if op == "_MatMulHeads":
        return _exec_matmul_heads(node, inp)
    if op == "_SoftmaxScaledMasked":
        return _exec_softmax_fused(node, inp)
    if op == "_FusedMatMulGelu":
        return _exec_matmul_gelu(node, inp)
    if op == "_FusedAttention":
        return _exec_fused_attention(node, inp)
    if op in ("FusedBatchNorm", "FusedBatchNormV2", "FusedBatchNormV3"):
        return ops.batch_norm(inp[0], inp[3], inp[4], inp[2], inp[1],
                              attr_number(node.attrs, "epsilon", 0.001))
    raise ValueError("Node type %s is not implemented" % op)


# ------------------------------------------------------------- plan rewrites --
def _exec_layer_norm(node, inp):
    eps = attr_number(node.attrs, "epsilon")
    from .kernels.reduce import layer_norm_supported
    tmp = []

    def keep(t):
        tmp.append(t)
        return t
    try:
        if attr_bool(node.attrs, "residual"):
            # the normalised tensor is Add(a, b), absorbed when both have its shape
            a, b, gamma, beta = inp
            if (a.dtype == "float32" and b.dtype == "float32" and
                    list(a.shape) == list(b.shape) and
                    layer_norm_supported(a.shape, gamma.shape, beta.shape)):
                return ops.fused_layer_norm(a, gamma, beta, eps, residual=b)
            x = keep(ops.add(a, b))
        else:
            x, gamma, beta = inp
        if x.dtype == "float32" and layer_norm_supported(x.shape, gamma.shape, beta.shape):
            return ops.fused_layer_norm(x, gamma, beta, eps)
        # shapes the one-launch kernel does not take: the matched subgraph, op by op
        mean = keep(ops.mean(x, [-1], True))
        var = keep(ops.mean(keep(ops.squared_difference(x, mean)), [-1], True))
        e = keep(ops.tensor(np.float32(eps)))
        rs = keep(ops.rsqrt(keep(ops.add(var, e))))
        norm = keep(ops.mul(keep(ops.sub(x, mean)), rs))
        return ops.add(keep(ops.mul(norm, gamma)), beta)
    finally:
        for t in tmp:
            t.dispose()


def fuse_layer_norms(ordered, is_const, const_value, const_shape, protected=()):
    """Plan rewrite in the spirit of the converter's graph fusions (FusedConv2D, _FusedMatMul
    are made the same way at conversion time): the subgraph a converted model holds for a
    layer normalisation over the last axis,

        mean = Mean(x, [-1], keep_dims); var = Mean(SquaredDifference(x, mean), [-1], keep_dims)
        out = AddV2(Mul(Mul(Sub(x, mean), Rsqrt(AddV2(var, eps))), gamma), beta)

    becomes one `_FusedLayerNorm(x, gamma, beta; epsilon)` node that keeps the name of `out`.
    Only when every intermediate is consumed inside the subgraph and none is in `protected`
    (requested outputs, fed inputs).  When x itself is an Add / AddV2 that nothing else
    consumes (the residual connection in front of the normalisation), it is absorbed too:
    `_FusedLayerNorm(a, b, gamma, beta; epsilon, residual)`.  `ordered` is a topologically sorted node list;
    is_const(name), const_value(name) -> flat numpy array, const_shape(name) -> list.
    Returns the new list and the number of subgraphs replaced."""
    by_name = {n.name: n for n in ordered}
    consumers = {}
    for n in ordered:
        for i in n.inputs:
            consumers.setdefault(parse_node_name(i)[0], []).append(n.name)
    protected = set(protected)

    def node(inp, op=None):
        name, idx = parse_node_name(inp)
        n = by_name.get(name)
        if n is None or idx != 0 or (op is not None and n.op not in op):
            return None
        return n

    def split(n, want_a, want_b):
        """The two inputs of a commutative node as (a, b) with a matching want_a."""
        if len(n.inputs) != 2:
            return None
        for a, b in ((n.inputs[0], n.inputs[1]), (n.inputs[1], n.inputs[0])):
            if want_a(a) and want_b(b):
                return a, b
        return None

    def const(inp):
        name, idx = parse_node_name(inp)
        return idx == 0 and name in by_name and by_name[name].op == "Const" and is_const(name)

    def last_axis_mean(n):
        if n is None or n.op != "Mean" or len(n.inputs) != 2 or not attr_bool(n.attrs, "keep_dims"):
            return False
        if not const(n.inputs[1]):
            return False
        axes = [int(v) for v in const_value(parse_node_name(n.inputs[1])[0])]
        return axes == [-1]

    def only(name, users):
        return sorted(consumers.get(name, [])) == sorted(users) and name not in protected

    ADD = ("Add", "AddV2")
    removed, replaced = set(), {}
    for out in ordered:
        if out.op not in ADD:
            continue
        ab = split(out, lambda i: node(i, ("Mul",)) is not None, const)
        if not ab:
            continue
        m2, beta = node(ab[0]), ab[1]
        ab = split(m2, lambda i: node(i, ("Mul",)) is not None, const)
        if not ab:
            continue
        norm, gamma = node(ab[0]), ab[1]
        ab = split(norm, lambda i: node(i, ("Sub",)) is not None,
                   lambda i: node(i, ("Rsqrt",)) is not None)
        if not ab:
            continue
        sub, rs = node(ab[0]), node(ab[1])
        if len(sub.inputs) != 2:
            continue
        x_in, mean = sub.inputs[0], node(sub.inputs[1])
        if not last_axis_mean(mean) or mean.inputs[0] != x_in:
            continue
        add = node(rs.inputs[0], ADD)
        if add is None:
            continue
        ab = split(add, lambda i: last_axis_mean(node(i)), const)
        if not ab:
            continue
        var, eps = node(ab[0]), ab[1]
        sq = node(var.inputs[0], ("SquaredDifference",))
        if sq is None or sorted(sq.inputs) != sorted([x_in, mean.name]):
            continue
        eps_v = const_value(parse_node_name(eps)[0])
        g_shape = list(const_shape(parse_node_name(gamma)[0]))
        b_shape = list(const_shape(parse_node_name(beta)[0]))
        if len(eps_v) != 1 or len(g_shape) != 1 or g_shape != b_shape:
            continue
        inner = (mean, sq, var, add, rs, sub, norm, m2)
        if len(set(n.name for n in inner)) != len(inner) or any(n.name in removed for n in inner):
            continue
        if not (only(mean.name, [sq.name, sub.name]) and only(sq.name, [var.name]) and
                only(var.name, [add.name]) and only(add.name, [rs.name]) and
                only(rs.name, [norm.name]) and only(sub.name, [norm.name]) and
                only(norm.name, [m2.name]) and only(m2.name, [out.name])):
            continue
        removed.update(n.name for n in inner)
        attrs = {"epsilon": {"f": float(np.float32(eps_v[0]))}}
        ins = [x_in, gamma, beta]
        xn = node(x_in, ADD)
        if (xn is not None and len(xn.inputs) == 2 and xn.name not in removed and
                only(xn.name, [mean.name, sq.name, sub.name])):
            removed.add(xn.name)
            ins = [xn.inputs[0], xn.inputs[1], gamma, beta]
            attrs["residual"] = {"b": True}
        replaced[out.name] = Node({"name": out.name, "op": "_FusedLayerNorm", "input": ins,
                                   "attr": attrs})
    if not replaced:
        return list(ordered), 0
    return [replaced.get(n.name, n) for n in ordered if n.name not in removed], len(replaced)


def _exec_matmul_gelu(node, inp):
    """_FusedMatMul whose epilogue is the erf GELU the five following nodes spelled out."""
    bias, prelu, act, alpha = _fused_params(node, inp)
    p = attr_number_list(node.attrs, "_gelu")
    ta, tb = attr_bool(node.attrs, "transpose_a"), attr_bool(node.attrs, "transpose_b")
    from ._cabi import CudaError, UNSUPPORTED
    if act == "linear" and bias is not None:
        try:
            return ops.fused_mat_mul(inp[0], inp[1], ta, tb, bias, "gelu_erf", None, alpha,
                                     geluParams=p)
        except CudaError as e:
            if e.code != UNSUPPORTED:
                raise
    h = ops.fused_mat_mul(inp[0], inp[1], ta, tb, bias, act, prelu, alpha)
    tmp = [h]
    try:
        c, half, one = [ops.tensor(np.float32(v)) for v in p[:3]]
        tmp += [c, half, one]
        a = ops.div(h, c) if p[3] else ops.mul(h, c)
        tmp.append(a)
        e = ops.erf(a)
        tmp.append(e)
        s1 = ops.add(e, one)
        tmp.append(s1)
        m = ops.mul(h, half)
        tmp.append(m)
        return ops.mul(m, s1)
    finally:
        for t in tmp:
            t.dispose()


def fuse_gelu_into_matmul(ordered, is_const, const_value, protected=()):
    """Plan rewrite: h = _FusedMatMul(a, b, bias) (no activation) followed by the erf GELU a
    converted graph spells as Mul(Mul(h, half), AddV2(Erf(Mul(h, scale)), one)) (or
    Erf(RealDiv(h, scale))), with scalar constants and h consumed by those two products
    only, becomes that `_FusedMatMul` with the GELU as its epilogue (node op
    `_FusedMatMulGelu`, named like the final Mul).  The epilogue performs the same fp32
    operations on the same h, so the bits do not change."""
    by_name = {n.name: n for n in ordered}
    consumers = {}
    for n in ordered:
        for i in n.inputs:
            consumers.setdefault(parse_node_name(i)[0], []).append(n.name)
    protected = set(protected)

    def node(inp, op):
        name, idx = parse_node_name(inp)
        n = by_name.get(name)
        return n if n is not None and idx == 0 and n.op in op else None

    def scalar_const(inp):
        name, idx = parse_node_name(inp)
        if idx != 0 or name not in by_name or by_name[name].op != "Const" or not is_const(name):
            return None
        v = const_value(name)
        return float(np.float32(v[0])) if len(v) == 1 else None

    def with_const(n, commutative=True):
        """(other input, constant) of a two-input node one of whose inputs is a scalar const."""
        if n is None or len(n.inputs) != 2:
            return None
        pairs = [(n.inputs[0], n.inputs[1])] + ([(n.inputs[1], n.inputs[0])] if commutative else [])
        for a, b in pairs:
            c = scalar_const(b)
            if c is not None and scalar_const(a) is None:
                return a, c
        return None

    def users(name):
        return sorted(consumers.get(name, []))

    removed, replaced = set(), {}
    for out in ordered:
        if out.op != "Mul" or len(out.inputs) != 2:
            continue
        for mi, ai in ((out.inputs[0], out.inputs[1]), (out.inputs[1], out.inputs[0])):
            m2, add = node(mi, ("Mul",)), node(ai, ("Add", "AddV2"))
            hm = with_const(m2)
            ea = with_const(add)
            if hm is None or ea is None:
                continue
            erf = node(ea[0], ("Erf",))
            if erf is None:
                continue
            inner = node(erf.inputs[0], ("Mul", "RealDiv", "Div"))
            hs = with_const(inner, commutative=inner is not None and inner.op == "Mul")
            if hs is None or hs[0] != hm[0]:
                continue
            mm = node(hm[0], ("_FusedMatMul",))
            if mm is None or mm.name in removed:
                continue
            fused = attr_string_list(mm.attrs, "fused_ops", [])
            if [f.lower() for f in fused] != ["biasadd"] or attr_number(mm.attrs, "num_args", 0) != 1:
                continue
            gone = [mm, m2, add, erf, inner]
            if (users(mm.name) != sorted([m2.name, inner.name]) or users(m2.name) != [out.name] or
                    users(add.name) != [out.name] or users(erf.name) != [add.name] or
                    users(inner.name) != [erf.name] or any(n.name in protected for n in gone)):
                continue
            removed.update(n.name for n in gone)
            attrs = dict(mm.attrs)
            attrs["_gelu"] = {"list": {"f": [hs[1], hm[1], ea[1], 1.0 if inner.op != "Mul" else 0.0]}}
            replaced[out.name] = Node({"name": out.name, "op": "_FusedMatMulGelu",
                                       "input": list(mm.inputs), "attr": attrs})
            break
    if not replaced:
        return list(ordered), 0
    return [replaced.get(n.name, n) for n in ordered if n.name not in removed], len(replaced)


def _exec_softmax_fused(node, inp):
    from .kernels.reduce import softmax_mask_rows
    scale = attr_number(node.attrs, "_scale")
    x = inp[0]
    mask = inp[1] if len(inp) > 1 else None
    if x.dtype == "float32" and len(x.shape) >= 1 and (
            mask is None or (mask.dtype == "float32" and
                             softmax_mask_rows(x.shape, mask.shape) is not None)):
        return ops.softmax_scaled_masked(x, scale, mask)
    tmp = []
    try:
        if scale is not None:
            c = ops.tensor(np.float32(scale))
            tmp.append(c)
            x = ops.mul(x, c)
            tmp.append(x)
        if mask is not None:
            x = ops.add(x, mask)
            tmp.append(x)
        return ops.softmax(x)
    finally:
        for t in tmp:
            t.dispose()


def fuse_softmax_inputs(ordered, is_const, const_value, protected=()):
    """Plan rewrite: Softmax(AddV2(Mul(s, c), mask)) and Softmax(Mul(s, c)) with c a scalar
    constant (attention scores scaled by 1 / sqrt(d) and masked) become one
    `_SoftmaxScaledMasked(s[, mask]; scale)` node named like the Softmax, when the
    intermediate tensors have no other consumer and are not in `protected`."""
    by_name = {n.name: n for n in ordered}
    consumers = {}
    for n in ordered:
        for i in n.inputs:
            consumers.setdefault(parse_node_name(i)[0], []).append(n.name)
    protected = set(protected)

    def node(inp, op):
        name, idx = parse_node_name(inp)
        n = by_name.get(name)
        return n if n is not None and idx == 0 and n.op in op else None

    def scalar_const(inp):
        name, idx = parse_node_name(inp)
        if idx != 0 or name not in by_name or by_name[name].op != "Const" or not is_const(name):
            return None
        v = const_value(name)
        return float(np.float32(v[0])) if len(v) == 1 else None

    def scaled(inp):
        """(scores input, scale, Mul node) when inp is Mul(scores, scalar const)."""
        m = node(inp, ("Mul",))
        if m is None or len(m.inputs) != 2:
            return None
        for a, b in ((m.inputs[0], m.inputs[1]), (m.inputs[1], m.inputs[0])):
            c = scalar_const(b)
            if c is not None and scalar_const(a) is None:
                return a, c, m
        return None

    def only(n, user):
        return consumers.get(n.name, []) == [user.name] and n.name not in protected

    removed, replaced = set(), {}
    for sm in ordered:
        if sm.op != "Softmax" or len(sm.inputs) != 1:
            continue
        ins, scale, gone = None, None, []
        add = node(sm.inputs[0], ("Add", "AddV2"))
        if add is not None and len(add.inputs) == 2 and only(add, sm):
            for a, b in ((add.inputs[0], add.inputs[1]), (add.inputs[1], add.inputs[0])):
                sc = scaled(a)
                if sc is not None and only(sc[2], add):
                    ins, scale, gone = [sc[0], b], sc[1], [add, sc[2]]
                    break
        else:
            sc = scaled(sm.inputs[0])
            if sc is not None and only(sc[2], sm):
                ins, scale, gone = [sc[0]], sc[1], [sc[2]]
        if ins is None:
            continue
        removed.update(n.name for n in gone)
        replaced[sm.name] = Node({"name": sm.name, "op": "_SoftmaxScaledMasked", "input": ins,
                                  "attr": {"_scale": {"f": scale}}})
    if not replaced:
        return list(ordered), 0
    return [replaced.get(n.name, n) for n in ordered if n.name not in removed], len(replaced)


_HEADS_REFUSED = set()   # (layout, operand shapes) the library has declined once


def _exec_matmul_heads(node, inp):
    """matMul + Reshape + Transpose([0, 2, 1, 3]) (heads split) or matMul + Transpose +
    Reshape (heads merged) as one product stored in the permuted order; the three ops one
    after the other when the library declines the shape."""
    from ._cabi import CudaError, UNSUPPORTED
    layout = attr_string(node.attrs, "_layout")
    inner_op = attr_string(node.attrs, "_op", keep_case=True)
    dims = attr_number_list(node.attrs, "_dims")      # the Reshape's target shape
    inner = Node({"name": node.name, "op": inner_op, "input": [], "attr": node.attrs})
    a, b = inp[0], inp[1]
    if inner_op == "_FusedMatMul":
        bias, prelu, act, alpha = _fused_params(inner, inp)
        ta, tb = attr_bool(node.attrs, "transpose_a"), attr_bool(node.attrs, "transpose_b")
    else:
        bias = prelu = alpha = None
        act = "linear"
        key = ("adj_x", "adj_y") if inner_op.startswith("BatchMatMul") else \
            ("transpose_a", "transpose_b")
        ta, tb = attr_bool(node.attrs, key[0]), attr_bool(node.attrs, key[1])
    if layout == "split":
        heads = dims if len(dims) == 4 and all(d > 0 for d in dims) else None
    else:
        # the product is [B, H, S, D]; the Reshape flattens its transpose [B, S, H, D]
        heads = None
        if len(a.shape) == 4 and len(b.shape) == 4:
            B, H = a.shape[0], a.shape[1]
            S = a.shape[2] if not ta else a.shape[3]
            D = b.shape[3] if not tb else b.shape[2]
            heads = [B, S, H, D]
    sig = (layout, tuple(a.shape), tuple(b.shape), ta, tb)
    if heads is not None and sig not in _HEADS_REFUSED:
        try:
            y = ops.mat_mul_heads(a, b, layout, heads, ta, tb, bias, act, prelu, alpha)
            if layout == "split":
                return y
            out = ops.reshape(y, dims)
            y.dispose()
            return out
        except CudaError as e:
            if e.code != UNSUPPORTED:
                raise
            _HEADS_REFUSED.add(sig)
    y = execute_op(inner, inp)
    try:
        if layout == "split":
            r = ops.reshape(y, dims)
            try:
                return ops.transpose(r, [0, 2, 1, 3])
            finally:
                r.dispose()
        t = ops.transpose(y, [0, 2, 1, 3])
        try:
            return ops.reshape(t, dims)
        finally:
            t.dispose()
    finally:
        y.dispose()


def fuse_attention_heads(ordered, is_const, const_value, protected=()):
    """Plan rewrite: the Reshape + Transpose([0, 2, 1, 3]) that splits a projection into
    attention heads, and the Transpose + Reshape that merges them again, become the store
    order of the product in front of them:

        Transpose(Reshape(matMul(a, b ...), [B, S, H, D]), [0, 2, 1, 3])  -> `_MatMulHeads` split
        Reshape(Transpose(batchMatMul(a, b), [0, 2, 1, 3]), shape)        -> `_MatMulHeads` merge

    when the intermediate tensors have no other consumer and are not in `protected`.  The
    new node keeps the name of the last node of the pattern and the attributes of the
    product."""
    by_name = {n.name: n for n in ordered}
    consumers = {}
    for n in ordered:
        for i in n.inputs:
            consumers.setdefault(parse_node_name(i)[0], []).append(n.name)
    protected = set(protected)
    MATMULS = ("_FusedMatMul", "MatMul", "BatchMatMul", "BatchMatMulV2")

    def node(inp, op):
        name, idx = parse_node_name(inp)
        n = by_name.get(name)
        return n if n is not None and idx == 0 and n.op in op else None

    def const_ints(inp):
        name, idx = parse_node_name(inp)
        if idx != 0 or name not in by_name or by_name[name].op != "Const" or not is_const(name):
            return None
        return [int(v) for v in const_value(name)]

    def only(n, user):
        return consumers.get(n.name, []) == [user.name] and n.name not in protected

    removed, replaced = set(), {}
    for last in ordered:
        if last.op == "Transpose" and len(last.inputs) == 2:            # heads split
            r = node(last.inputs[0], ("Reshape",))
            mm = node(r.inputs[0], MATMULS) if r is not None and len(r.inputs) == 2 else None
            if mm is None or const_ints(last.inputs[1]) != [0, 2, 1, 3]:
                continue
            dims = const_ints(r.inputs[1])
            layout = "split"
            mid = r
        elif last.op == "Reshape" and len(last.inputs) == 2:            # heads merge
            t = node(last.inputs[0], ("Transpose",))
            mm = node(t.inputs[0], MATMULS) if t is not None and len(t.inputs) == 2 else None
            if mm is None or const_ints(t.inputs[1]) != [0, 2, 1, 3]:
                continue
            dims = const_ints(last.inputs[1])
            layout = "merge"
            mid = t
        else:
            continue
        if dims is None or any(d <= 0 for d in dims) or (layout == "split" and len(dims) != 4):
            continue
        if mm.name in removed or not only(mm, mid) or not only(mid, last):
            continue
        removed.update((mm.name, mid.name))
        attrs = dict(mm.attrs)
        attrs["_layout"] = {"s": base64.b64encode(layout.encode()).decode()}
        attrs["_op"] = {"s": base64.b64encode(mm.op.encode()).decode()}
        attrs["_dims"] = {"list": {"i": [str(d) for d in dims]}}
        replaced[last.name] = Node({"name": last.name, "op": "_MatMulHeads",
                                    "input": list(mm.inputs), "attr": attrs})
    if not replaced:
        return list(ordered), 0
    return [replaced.get(n.name, n) for n in ordered if n.name not in removed], len(replaced)


_ATTENTION_REFUSED = set()   # operand shapes the library has declined once


def _exec_fused_attention(node, inp):
    """softmax(q k^T * scale + mask) v stored with the heads merged, as one launch; the
    batched product, the scaled, masked softmax and the heads-merging product one after the
    other when the library declines the shape."""
    from ._cabi import CudaError, UNSUPPORTED
    q, k, v = inp[0], inp[1], inp[2]
    mask = inp[3] if len(inp) > 3 else None
    scale = attr_number(node.attrs, "_scale")
    dims = attr_number_list(node.attrs, "_dims")
    sig = (tuple(q.shape), tuple(k.shape), tuple(v.shape),
           tuple(mask.shape) if mask is not None else None)
    if sig not in _ATTENTION_REFUSED:
        try:
            y = ops.fused_attention(q, k, v, scale, mask)
            try:
                return ops.reshape(y, dims)
            finally:
                y.dispose()
        except CudaError as e:
            if e.code != UNSUPPORTED:
                raise
            _ATTENTION_REFUSED.add(sig)
    scores = ops.mat_mul(q, k, False, True)
    try:
        attrs = {} if scale is None else {"_scale": {"f": scale}}
        sm = Node({"name": node.name, "op": "_SoftmaxScaledMasked", "input": [], "attr": attrs})
        probs = _exec_softmax_fused(sm, [scores] if mask is None else [scores, mask])
    finally:
        scores.dispose()
    try:
        enc = lambda t: {"s": base64.b64encode(t.encode()).decode()}
        merge = Node({"name": node.name, "op": "_MatMulHeads", "input": [],
                      "attr": {"_layout": enc("merge"), "_op": enc("BatchMatMulV2"),
                               "_dims": node.attrs["_dims"]}})
        return _exec_matmul_heads(merge, [probs, v])
    finally:
        probs.dispose()


def fuse_attention(ordered, protected=()):
    """Plan rewrite: the heads-merging product of softmax(scores) and v, with scores =
    batchMatMul(q, k, adj_y) (scaled and masked on the way into the softmax or not), becomes
    one `_FusedAttention(q, k, v[, mask]; scale)` node named like the merge, when the scores
    and the probabilities have no other consumer and are not in `protected`.  Runs after
    fuse_attention_heads and fuse_softmax_inputs, whose nodes it matches."""
    by_name = {n.name: n for n in ordered}
    consumers = {}
    for n in ordered:
        for i in n.inputs:
            consumers.setdefault(parse_node_name(i)[0], []).append(n.name)
    protected = set(protected)

    def node(inp, op):
        name, idx = parse_node_name(inp)
        n = by_name.get(name)
        return n if n is not None and idx == 0 and n.op in op else None

    def only(n, user):
        return consumers.get(n.name, []) == [user.name] and n.name not in protected

    removed, replaced = set(), {}
    for last in ordered:
        if last.op != "_MatMulHeads" or attr_string(last.attrs, "_layout") != "merge" or \
                len(last.inputs) != 2:
            continue
        if not attr_string(last.attrs, "_op", keep_case=True).startswith("BatchMatMul") or \
                attr_bool(last.attrs, "adj_x") or attr_bool(last.attrs, "adj_y"):
            continue
        sm = node(last.inputs[0], ("_SoftmaxScaledMasked", "Softmax"))
        if sm is None or not only(sm, last) or not 1 <= len(sm.inputs) <= 2:
            continue
        sc = node(sm.inputs[0], ("BatchMatMul", "BatchMatMulV2"))
        if sc is None or len(sc.inputs) != 2 or not only(sc, sm) or \
                attr_bool(sc.attrs, "adj_x") or not attr_bool(sc.attrs, "adj_y"):
            continue
        attrs = {"_dims": last.attrs["_dims"]}
        if sm.op == "_SoftmaxScaledMasked" and "_scale" in sm.attrs:
            attrs["_scale"] = sm.attrs["_scale"]
        removed.update((sc.name, sm.name))
        replaced[last.name] = Node({"name": last.name, "op": "_FusedAttention",
                                    "input": [sc.inputs[0], sc.inputs[1], last.inputs[1]] +
                                             list(sm.inputs[1:]),
                                    "attr": attrs})
    if not replaced:
        return list(ordered), 0
    return [replaced.get(n.name, n) for n in ordered if n.name not in removed], len(replaced)


def hoist_shared_operand_matmuls(ordered, is_const):
    """Plan rewrite (scheduling only): products whose first operand is the same tensor and
    whose other operands are constants run next to each other.  The backend launches the
    products pending on one operand as a group; in the stored order of an attention layer
    the value projection comes after the softmax and would miss the group of the query and
    key projections."""
    MATMULS = ("_FusedMatMul", "MatMul", "_MatMulHeads")
    first, moved = {}, {}
    for n in ordered:
        if n.op not in MATMULS or len(n.inputs) < 2:
            continue
        if not all(is_const(parse_node_name(i)[0]) for i in n.inputs[1:]):
            continue
        a = n.inputs[0]
        if a in first:
            moved.setdefault(first[a], []).append(n)
        else:
            first[a] = n.name
    if not moved:
        return list(ordered), 0
    late = set(m.name for ms in moved.values() for m in ms)
    by_name = {n.name: n for n in ordered}
    out, placed = [], set()
    for n in ordered:
        if n.name in late or n.name in placed:
            continue
        out.append(n)
        placed.add(n.name)
        for m in moved.get(n.name, ()):
            # the constants a moved product reads must precede it
            for i in m.inputs[1:]:
                cname = parse_node_name(i)[0]
                if cname not in placed and cname in by_name:
                    out.append(by_name[cname])
                    placed.add(cname)
            out.append(m)
            placed.add(m.name)
    return out, len(late)


# ------------------------------------------------------------------- executor --
class GraphExecutor(object):
    def __init__(self, nodes, weight_map):
        self.nodes = {n.name: n for n in nodes}
        self.order_all = nodes
        self.weight_map = weight_map      # name -> Tensor (kept for the model's lifetime)
        self.placeholders = [n for n in nodes if n.op == "Placeholder"]
        consumed = set()
        for n in nodes:
            for i in n.inputs:
                consumed.add(parse_node_name(i)[0])
        self.default_outputs = [n.name for n in nodes
                                if n.name not in consumed and n.op not in ("Const", "Placeholder")]
        self._compiled = {}
        # plan rewrites (fuse_layer_norms); TFJS_CUDA_NO_GRAPH_FUSION=1 runs the graph as stored
        off = os.environ.get("TFJS_CUDA_NO_GRAPH_FUSION", "0")
        self.fuse = off in ("", "0") or off not in ("1", "all")
        # ...=layernorm,heads,softmax switches single rewrites off
        self.fuse_skip = set(off.split(",")) if self.fuse else set()
        self.fused_subgraphs = 0
        self.fused_heads = 0
        self.fused_softmaxes = 0
        self.fused_gelus = 0
        self.fused_attentions = 0
        self.hoisted_matmuls = 0
        self.keep_intermediates = False
        self.intermediates = {}

    def _compile(self, input_names, output_names):
        """graph_executor.ts:167-191: the nodes needed for the outputs in topological
        order, and for every tensor the position of its last consumer."""
        fuse = self.fuse and not self.keep_intermediates
        key = (tuple(sorted(input_names)), tuple(output_names), fuse)
        if key in self._compiled:
            return self._compiled[key]
        needed, stack = set(), [parse_node_name(o)[0] for o in output_names]
        while stack:
            name = stack.pop()
            if name in needed:
                continue
            if name not in self.nodes:
                raise ValueError("The output '%s' is not found in the graph" % name)
            needed.add(name)
            if name in input_names:
                continue
            stack.extend(parse_node_name(i)[0] for i in self.nodes[name].inputs)
        for name in needed:
            n = self.nodes[name]
            if n.op == "Placeholder" and name not in input_names:
                raise ValueError("Cannot compute the outputs [%s] from the provided inputs [%s]. "
                                 "Missing the following inputs: [%s]" %
                                 (", ".join(output_names), ", ".join(input_names), name))
        ordered, state = [], {}

        def visit(name):
            # iterative DFS post-order
            st = [(name, 0)]
            while st:
                cur, idx = st.pop()
                if state.get(cur) == 2:
                    continue
                node = self.nodes[cur]
                ins = [] if cur in input_names else [parse_node_name(i)[0] for i in node.inputs]
                if idx < len(ins):
                    st.append((cur, idx + 1))
                    if state.get(ins[idx]) is None:
                        state[ins[idx]] = 1
                        st.append((ins[idx], 0))
                else:
                    state[cur] = 2
                    ordered.append(node)
        for o in output_names:
            root = parse_node_name(o)[0]
            if state.get(root) is None:
                state[root] = 1
                visit(root)
        if fuse:
            n = k = j = 0
            prot = set(input_names) | set(parse_node_name(o)[0] for o in output_names)
            consts = (lambda name: name in self.weight_map,
                      lambda name: np.asarray(_vals(self.weight_map[name])).reshape(-1))
        if fuse and "layernorm" not in self.fuse_skip:
            ordered, n = fuse_layer_norms(
                ordered, lambda name: name in self.weight_map,
                lambda name: np.asarray(_vals(self.weight_map[name])).reshape(-1),
                lambda name: self.weight_map[name].shape,
                protected=set(input_names) | set(parse_node_name(o)[0] for o in output_names))
        if fuse and "heads" not in self.fuse_skip:
            ordered, k = fuse_attention_heads(ordered, consts[0], consts[1], protected=prot)
        # The erf GELU behind a dense layer becomes that product's epilogue (its packed fp32
        # evaluation fits beside the main loop: +11 us on the [8192, 768] x [768, 3072]
        # product against 35 us for the chain kernel); TFJS_CUDA_NO_FUSE_GELU=1 keeps the chain.
        if fuse and "gelu" not in self.fuse_skip and \
                os.environ.get("TFJS_CUDA_NO_FUSE_GELU", "0") in ("", "0"):
            ordered, self.fused_gelus = fuse_gelu_into_matmul(ordered, consts[0], consts[1],
                                                              protected=prot)
        if fuse and "softmax" not in self.fuse_skip:
            ordered, j = fuse_softmax_inputs(ordered, consts[0], consts[1], protected=prot)
        if fuse and "attention" not in self.fuse_skip:
            ordered, self.fused_attentions = fuse_attention(ordered, protected=prot)
        if fuse and "hoist" not in self.fuse_skip:
            ordered, self.hoisted_matmuls = hoist_shared_operand_matmuls(ordered, consts[0])
        if fuse:
            self.fused_subgraphs = n
            self.fused_heads = k
            self.fused_softmaxes = j
        last_use = {}
        for pos, node in enumerate(ordered):
            if node.name in input_names:
                continue
            for i in node.inputs:
                last_use[parse_node_name(i)[0]] = pos
        plan = (ordered, last_use)
        self._compiled[key] = plan
        return plan

    def execute(self, inputs, outputs=None):
        """graph_executor.ts:231-318."""
        outputs = list(outputs) if outputs else list(self.default_outputs)
        input_names = set(inputs)
        for name, t in inputs.items():
            node = self.nodes.get(name)
            if node is None:
                raise ValueError("The dict provided in model.execute(dict) has keys: [%s] that "
                                 "are not part of graph" % name)
            shape = attr_shape(node.attrs, "shape")
            if shape is not None:
                ok = len(shape) == len(t.shape) and all(
                    s in (-1, d) for s, d in zip(shape, t.shape))
                if not ok:
                    raise ValueError("The shape of dict['%s'] provided in model.execute(dict) must "
                                     "be [%s], but was [%s]" % (name, shape, t.shape))
            dt = attr_dtype(node.attrs, "dtype")
            if dt is not None and dt != t.dtype:
                raise ValueError("The dtype of dict['%s'] provided in model.execute(dict) must be "
                                 "%s, but was %s" % (name, dt, t.dtype))
        ordered, last_use = self._compile(input_names, outputs)
        out_roots = set(parse_node_name(o)[0] for o in outputs)
        tensors = {}
        owned = set()
        self.intermediates = {}
        try:
            for pos, node in enumerate(ordered):
                if node.name in input_names:
                    tensors[node.name] = inputs[node.name]
                elif node.op == "Const":
                    tensors[node.name] = self.weight_map[node.name]
                else:
                    ins = [tensors[parse_node_name(i)[0]] for i in node.inputs]
                    tensors[node.name] = execute_op(node, ins)
                    owned.add(node.name)
                # dispose what nobody downstream needs (graph_executor.ts:382-409)
                if not self.keep_intermediates and node.name not in input_names:
                    for i in node.inputs:
                        src = parse_node_name(i)[0]
                        if (src in owned and last_use.get(src) == pos and src not in out_roots):
                            tensors[src].dispose()
                            owned.discard(src)
            result = [tensors[parse_node_name(o)[0]] for o in outputs]
        except Exception:
            for name in owned:
                tensors[name].dispose()
            raise
        if self.keep_intermediates:
            self.intermediates = {n: tensors[n] for n in owned}
        else:
            for name in list(owned):
                if name not in out_roots:
                    tensors[name].dispose()
        return result


class GraphModel(object):
    """tfjs-converter/src/executor/graph_model.ts."""

    def __init__(self, model_json, weight_data, engine=None, decode_weights=None, replay=None):
        self.engine = engine or ENGINE
        # Whole-step replay: after one eager execute per (input shapes, outputs) signature
        # the step is captured into a CUDA graph and later executes are one launch.
        self.replay = (os.environ.get("TFJS_CUDA_GRAPH_REPLAY", "0") not in ("", "0")
                       if replay is None else bool(replay))
        self._replays = {}
        self.artifacts = model_json if isinstance(model_json, dict) else json.loads(model_json)
        if self.artifacts.get("format") not in (None, "graph-model"):
            raise ValueError("not a graph-model artifact")
        topo = self.artifacts["modelTopology"]
        if "versions" not in topo:
            raise ValueError("modelTopology.versions is missing")
        self.version = "%s.%s" % (topo["versions"].get("producer"),
                                  topo["versions"].get("minConsumer"))
        specs = []
        for group in self.artifacts.get("weightsManifest", []):
            specs.extend(group["weights"])
        # weights go through the library's loader (pinned staging, device-side decode);
        # io.decode_weights is the per-tensor path with the same results
        decode = decode_weights or io.load_weights
        self.weights = decode(self.engine, weight_data, specs)
        nodes = [Node(d) for d in topo["node"]]
        for n in nodes:
            if n.op == "Const" and n.name not in self.weights:
                raise ValueError("Const node %s has no weight in the manifest" % n.name)
        self.executor = GraphExecutor(nodes, self.weights)
        sig = (self.artifacts.get("userDefinedMetadata") or {}).get("signature") or \
            self.artifacts.get("signature") or {}
        self.input_names = list((sig.get("inputs") or {}).keys()) or \
            [n.name for n in self.executor.placeholders]
        self.output_names = list((sig.get("outputs") or {}).keys()) or \
            self.executor.default_outputs

    @classmethod
    def load(cls, model_json_path, engine=None, replay=None):
        """tf.loadGraphModel for a model.json on disk: the weight shards named by
        weightsManifest[].paths (relative to the model.json) are read by the library itself
        (graph_model.ts:176-234 with the file handler of tfjs-node's io)."""
        with open(model_json_path) as f:
            artifacts = json.load(f)
        base = os.path.dirname(os.path.abspath(model_json_path))
        eng = engine or ENGINE

        def from_files(engine_, _unused, specs):
            paths = []
            for group in artifacts.get("weightsManifest", []):
                paths.extend(os.path.join(base, p) for p in group["paths"])
            return io.load_weights_from_files(engine_, paths, specs)
        return cls(artifacts, None, eng, decode_weights=from_files, replay=replay)

    @property
    def inputs(self):
        return [{"name": n.name, "shape": attr_shape(n.attrs, "shape"),
                 "dtype": attr_dtype(n.attrs, "dtype")} for n in self.executor.placeholders]

    def execute(self, inputs, outputs=None):
        """graph_model.ts:507-516: inputs is a Tensor, a list, or a name->Tensor dict."""
        if isinstance(inputs, Tensor):
            inputs = [inputs]
        if isinstance(inputs, (list, tuple)):
            if len(inputs) != len(self.input_names):
                raise ValueError("Input tensor count mismatch, the graph model has %d "
                                 "placeholders, while there are %d input tensors." %
                                 (len(self.input_names), len(inputs)))
            inputs = dict(zip(self.input_names, inputs))
        single = isinstance(outputs, str) or (outputs is None and len(self.output_names) == 1)
        if isinstance(outputs, str):
            outputs = [outputs]
        outputs = outputs or self.output_names
        if self.replay and self.engine._profile is None and not self.executor.keep_intermediates:
            res = self._execute_replayed(inputs, list(outputs))
        else:
            res = self.executor.execute(inputs, outputs)
        return res[0] if single else res

    # ------------------------------------------------------------ step replay --
    def _execute_replayed(self, inputs, outputs):
        """First call per signature: eager, measuring the step's peak memory.  Second:
        the executor runs once more under stream capture (nothing executes; every kernel
        call is recorded, intermediates live in an arena owned by the graph).  From then
        on: copy the inputs into the captured input buffers, launch the graph, copy the
        outputs out.  A step that cannot be captured (a kernel that needs the host)
        stays eager."""
        from ._cabi import CudaError, UNSUPPORTED
        be = self.engine.backend
        key = (tuple(sorted((n, tuple(t.shape), t.dtype) for n, t in inputs.items())),
               tuple(outputs))
        st = self._replays.get(key)
        if st is None:
            be.high_water_reset()
            before = be.memory()["numBytesInGPU"]
            res = self.executor.execute(inputs, outputs)
            for t in res:
                be.device_id(t.dataId)          # launch anything still pending
            peak = be.memory()["poolHighWater"] - before
            self._replays[key] = {"state": "warm", "peak": max(int(peak), 0)}
            return res
        if st["state"] == "warm":
            try:
                self._capture(st, inputs, outputs)
                st["state"] = "ready"
            except CudaError as e:
                if "arena" in str(e) and st.get("arena_retries", 0) < 2:
                    # the arena (sized from the eager step's peak) fragmented: this step runs
                    # eagerly and the next one captures with more room
                    st["arena_retries"] = st.get("arena_retries", 0) + 1
                    st["peak"] = int(st["peak"] * 1.6) + (64 << 20)
                else:
                    st["state"] = "eager"
                st["why"] = str(e)
        if st["state"] != "ready":
            return self.executor.execute(inputs, outputs)
        for name, t in inputs.items():
            be.copy(t.dataId, st["fixed"][name].dataId)
        try:
            be.graph_launch(st["graph"])
        except CudaError as e:
            if e.code != UNSUPPORTED:
                raise
            # the graph went stale (a weight it reads was freed or rewritten, or the
            # library's scratch buffer moved): drop it, run this step eagerly, and let the
            # next execute of this signature capture again
            self._drop_replay(st)
            again = st.get("recaptures", 0) + 1
            st.clear()
            # a step that keeps going stale is not worth capturing
            st.update(state="warm" if again <= 3 else "eager", peak=0, recaptures=again,
                      why="captured step went stale %d times" % again)
            be.high_water_reset()
            before = be.memory()["numBytesInGPU"]
            res = self.executor.execute(inputs, outputs)
            for t in res:
                be.device_id(t.dataId)
            st["peak"] = max(int(be.memory()["poolHighWater"] - before), 0)
            return res
        res = []
        for o in st["outs"]:
            fresh = be.make_output(o.shape, o.dtype)
            be.copy(o.dataId, fresh.dataId)
            res.append(self.engine.make_tensor_from_info(fresh))
        return res

    def _capture(self, st, inputs, outputs):
        be, eng = self.engine.backend, self.engine
        fixed = {}
        for name, t in inputs.items():
            info = be.make_output(t.shape, t.dtype)
            fixed[name] = eng.make_tensor_from_info(info)
            be.copy(t.dataId, info.dataId)
        outs = None
        be.capture_begin(int(st["peak"] * 1.25) + (4 << 20))
        try:
            outs = self.executor.execute(fixed, outputs)
            for t in outs:
                be.device_id(t.dataId)
            st["graph"] = be.capture_end(False)
        except Exception:
            try:
                be.capture_end(True)
            except Exception:
                pass
            for t in (outs or []):
                t.dispose()
            for t in fixed.values():
                t.dispose()
            raise
        st["fixed"], st["outs"] = fixed, outs

    def predict(self, inputs):
        return self.execute(inputs)

    def _drop_replay(self, st):
        if st.get("state") == "ready":
            for t in st["outs"]:
                t.dispose()
            for t in st["fixed"].values():
                t.dispose()
            self.engine.backend.graph_destroy(st["graph"])

    def dispose(self):
        for st in self._replays.values():
            self._drop_replay(st)
        self._replays = {}
        for t in self.weights.values():
            t.dispose()
        self.weights = {}
