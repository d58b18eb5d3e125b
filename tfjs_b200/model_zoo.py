"""Synthetic graph-model artifacts (model.json + weight bytes) for the benchmark
configurations: MobileNetV2-1.0, ResNet-50 v1.5 and a BERT-base-shaped encoder.

The artifacts use the converter's wire format (tfjs-core/src/io/types.ts:49-110;
node attribute encoding as read by tfjs-converter/src/operations/
operation_mapper.ts:437-461: ints are JSON strings, strings are base64), with the
op set the converter emits after its grappler passes: `_FusedConv2D` and
`FusedDepthwiseConv2dNative` with BiasAdd + activation, `_FusedMatMul`,
`BatchMatMulV2`, `AddV2`, `Mean`, `MaxPool`, ...  Weights are random-initialised
(there are no pretrained checkpoints offline); BatchNorm is folded into the
convolution bias.  The same artifacts load in an unmodified GraphModel.
"""
import base64

import numpy as np


def _s(text):
    return {"s": base64.b64encode(text.encode()).decode()}


def _i(v):
    return {"i": str(int(v))}


def _ilist(vals):
    return {"list": {"i": [str(int(v)) for v in vals]}}


def _slist(vals):
    return {"list": {"s": [base64.b64encode(v.encode()).decode() for v in vals]}}


def _shape(shape):
    return {"shape": {"dim": [{"size": str(int(s))} for s in shape]}}


_ACT = {"relu": "Relu", "relu6": "Relu6", "elu": "Elu", "leakyrelu": "LeakyRelu",
        "sigmoid": "Sigmoid"}


class GraphBuilder(object):
    def __init__(self, seed=0):
        self.nodes = []
        self.weights = []          # (name, array) in manifest order
        self.rng = np.random.default_rng(seed)
        self._n = 0

    def _name(self, base):
        self._n += 1
        return "%s_%d" % (base, self._n)

    def node(self, op, inputs, attrs=None, name=None):
        name = name or self._name(op.strip("_").lower())
        self.nodes.append({"name": name, "op": op, "input": list(inputs), "attr": attrs or {}})
        return name

    def placeholder(self, name, shape, dtype="DT_FLOAT"):
        return self.node("Placeholder", [], {"dtype": {"type": dtype}, "shape": _shape(shape)},
                         name)

    def const(self, array, name=None):
        array = np.asarray(array)
        name = name or self._name("const")
        dt = "DT_INT32" if np.issubdtype(array.dtype, np.integer) else "DT_FLOAT"
        self.nodes.append({"name": name, "op": "Const", "input": [],
                           "attr": {"dtype": {"type": dt}, "value": {"tensor": {"dtype": dt}}}})
        self.weights.append((name, array))
        return name

    # ------------------------------------------------------------ layers ----
    def _fused_attrs(self, activation, extra):
        fused = ["BiasAdd"] + ([_ACT[activation]] if activation not in (None, "linear") else [])
        attrs = {"fused_ops": _slist(fused), "num_args": _i(1), "T": {"type": "DT_FLOAT"},
                 "epsilon": {"f": 0.0}, "leakyrelu_alpha": {"f": 0.2}}
        attrs.update(extra)
        return attrs

    def conv(self, x, w, b, stride=1, activation="relu", padding="SAME", name=None):
        return self.node("_FusedConv2D", [x, self.const(w), self.const(b)], self._fused_attrs(
            activation, {"strides": _ilist([1, stride, stride, 1]), "padding": _s(padding),
                         "dilations": _ilist([1, 1, 1, 1]), "data_format": _s("NHWC"),
                         "explicit_paddings": {"list": {}}, "use_cudnn_on_gpu": {"b": True}}), name)

    def depthwise(self, x, w, b, stride=1, activation="relu6", name=None):
        return self.node("FusedDepthwiseConv2dNative", [x, self.const(w), self.const(b)],
                         self._fused_attrs(activation, {
                             "strides": _ilist([1, stride, stride, 1]), "padding": _s("SAME"),
                             "dilations": _ilist([1, 1, 1, 1]), "data_format": _s("NHWC"),
                             "explicit_paddings": {"list": {}}}), name)

    def dense(self, x, w, b, activation=None, name=None):
        return self.node("_FusedMatMul", [x, self.const(w), self.const(b)], self._fused_attrs(
            activation, {"transpose_a": {"b": False}, "transpose_b": {"b": False}}), name)

    def binary(self, op, a, b, name=None):
        return self.node(op, [a, b], {"T": {"type": "DT_FLOAT"}}, name)

    def unary(self, op, x, name=None):
        return self.node(op, [x], {"T": {"type": "DT_FLOAT"}}, name)

    def mean(self, x, axes, keep_dims=False, name=None):
        return self.node("Mean", [x, self.const(np.asarray(axes, np.int32))],
                         {"keep_dims": {"b": bool(keep_dims)}, "T": {"type": "DT_FLOAT"},
                          "Tidx": {"type": "DT_INT32"}}, name)

    def max_pool(self, x, ksize, stride, padding="SAME", name=None):
        return self.node("MaxPool", [x], {"ksize": _ilist([1, ksize, ksize, 1]),
                                          "strides": _ilist([1, stride, stride, 1]),
                                          "padding": _s(padding), "data_format": _s("NHWC"),
                                          "T": {"type": "DT_FLOAT"}}, name)

    def reshape(self, x, shape, name=None):
        return self.node("Reshape", [x, self.const(np.asarray(shape, np.int32))],
                         {"T": {"type": "DT_FLOAT"}, "Tshape": {"type": "DT_INT32"}}, name)

    def transpose(self, x, perm, name=None):
        return self.node("Transpose", [x, self.const(np.asarray(perm, np.int32))],
                         {"T": {"type": "DT_FLOAT"}, "Tperm": {"type": "DT_INT32"}}, name)

    def batch_matmul(self, a, b, adj_x=False, adj_y=False, name=None):
        return self.node("BatchMatMulV2", [a, b], {"adj_x": {"b": adj_x}, "adj_y": {"b": adj_y},
                                                   "T": {"type": "DT_FLOAT"}}, name)

    def gather(self, params, indices, axis=0, name=None):
        return self.node("GatherV2", [params, indices, self.const(np.asarray(axis, np.int32))],
                         {"batch_dims": _i(0), "Tparams": {"type": "DT_FLOAT"},
                          "Tindices": {"type": "DT_INT32"}, "Taxis": {"type": "DT_INT32"}}, name)

    def layer_norm(self, x, gamma, beta, eps):
        """The decomposed form the converter leaves in a graph:
        (x - mean) * rsqrt(var + eps) * gamma + beta over the last axis."""
        mean = self.mean(x, [-1], True)
        sq = self.binary("SquaredDifference", x, mean)
        var = self.mean(sq, [-1], True)
        rs = self.unary("Rsqrt", self.binary("AddV2", var, self.const(np.float32(eps))))
        norm = self.binary("Mul", self.binary("Sub", x, mean), rs)
        return self.binary("AddV2", self.binary("Mul", norm, self.const(gamma)),
                           self.const(beta))

    # ------------------------------------------------------------- output ----
    def artifacts(self, inputs, outputs, quantize=None):
        from . import io
        weight_bytes, specs = io.encode_weights(self.weights, quantize)
        sig = {"inputs": {n: {"name": n + ":0"} for n in inputs},
               "outputs": {n: {"name": n + ":0"} for n in outputs}}
        model = {"format": "graph-model", "generatedBy": "tfjs_b200.model_zoo",
                 "convertedBy": "synthetic",
                 "modelTopology": {"node": self.nodes, "library": {},
                                   "versions": {"producer": 1395, "minConsumer": 12}},
                 "weightsManifest": [{"paths": ["group1-shard1of1.bin"], "weights": specs}],
                 "signature": sig}
        return model, weight_bytes


def _glorot(rng, shape, fan_in, fan_out):
    lim = np.sqrt(6.0 / (fan_in + fan_out))
    return rng.uniform(-lim, lim, shape).astype(np.float32)


def _he(rng, shape, fan_in):
    return (rng.standard_normal(shape) * np.sqrt(2.0 / fan_in)).astype(np.float32)


def mobilenet_v2(batch, size=224, alpha=1.0, classes=1000, seed=0, softmax=False):
    """MobileNetV2: 3x3/2 stem (32), 17 inverted-residual blocks (t,c,n,s) =
    (1,16,1,1),(6,24,2,2),(6,32,3,2),(6,64,4,2),(6,96,3,1),(6,160,3,2),(6,320,1,1),
    1x1 conv 1280, global average pool, dense.  Glorot-uniform weights; the folded
    BatchNorm shows up as a small per-channel bias N(0, 0.01)."""
    g = GraphBuilder(seed)
    r = g.rng
    bias = lambda c: (r.standard_normal(c) * 0.01).astype(np.float32)
    ch = lambda c: max(8, int(c * alpha + 4) // 8 * 8)
    x = g.placeholder("input", [batch, size, size, 3])
    c_in = ch(32)
    x = g.conv(x, _glorot(r, (3, 3, 3, c_in), 27, 9 * c_in), bias(c_in), 2, "relu6")
    for t, c, n, s in ((1, 16, 1, 1), (6, 24, 2, 2), (6, 32, 3, 2), (6, 64, 4, 2),
                       (6, 96, 3, 1), (6, 160, 3, 2), (6, 320, 1, 1)):
        c_out = ch(c)
        for i in range(n):
            stride = s if i == 0 else 1
            y = x
            c_mid = c_in * t
            if t != 1:
                y = g.conv(y, _glorot(r, (1, 1, c_in, c_mid), c_in, c_mid), bias(c_mid), 1, "relu6")
            y = g.depthwise(y, _glorot(r, (3, 3, c_mid, 1), 9, 9), bias(c_mid), stride, "relu6")
            y = g.conv(y, _glorot(r, (1, 1, c_mid, c_out), c_mid, c_out), bias(c_out), 1, None)
            if stride == 1 and c_in == c_out:
                y = g.binary("AddV2", x, y)
            x, c_in = y, c_out
    c_last = max(1280, ch(1280)) if alpha > 1.0 else 1280
    x = g.conv(x, _glorot(r, (1, 1, c_in, c_last), c_in, c_last), bias(c_last), 1, "relu6")
    x = g.mean(x, [1, 2])
    x = g.dense(x, _glorot(r, (c_last, classes), c_last, classes), bias(classes), None,
                name=None if softmax else "logits")
    if softmax:
        x = g.node("Softmax", [x], {"T": {"type": "DT_FLOAT"}}, "probs")
    return g.artifacts(["input"], [x])


def resnet50(batch, size=224, classes=1000, seed=0, quantize="uint8", width=64):
    """ResNet-50 v1.5: 7x7/2 stem, 3x3/2 max pool, bottleneck stages [3,4,6,3] with the
    stride on the 3x3 convolution, projection shortcut on the first block of each
    stage, Add then Relu, global average pool, dense.  He-normal weights, stored
    with the converter's per-tensor uint8 affine quantisation; biases stay float32."""
    g = GraphBuilder(seed)
    r = g.rng
    bias = lambda c: (r.standard_normal(c) * 0.01).astype(np.float32)
    x = g.placeholder("input", [batch, size, size, 3])
    x = g.conv(x, _he(r, (7, 7, 3, width), 147), bias(width), 2, "relu")
    x = g.max_pool(x, 3, 2)
    c_in = width
    for stage, blocks in enumerate((3, 4, 6, 3)):
        mid = width * (2 ** stage)
        out = mid * 4
        for b in range(blocks):
            stride = 2 if (b == 0 and stage > 0) else 1
            sc = x
            if b == 0:
                sc = g.conv(x, _he(r, (1, 1, c_in, out), c_in), bias(out), stride, None)
            y = g.conv(x, _he(r, (1, 1, c_in, mid), c_in), bias(mid), 1, "relu")
            y = g.conv(y, _he(r, (3, 3, mid, mid), 9 * mid), bias(mid), stride, "relu")
            y = g.conv(y, _he(r, (1, 1, mid, out), mid), bias(out), 1, None)
            x = g.unary("Relu", g.binary("AddV2", sc, y))
            c_in = out
    x = g.mean(x, [1, 2])
    x = g.dense(x, _he(r, (c_in, classes), c_in), bias(classes), None, name="logits")
    return g.artifacts(["input"], [x], quantize)


def bert_encoder(batch, seq=128, layers=12, hidden=768, heads=12, ffn=3072, vocab=30522,
                 max_pos=512, seed=0):
    """BERT-base-shaped encoder as a tfjs ops graph: word + position embeddings
    (GatherV2 + AddV2) -> LayerNorm; per layer Q/K/V/O dense, heads split with
    Reshape + Transpose, scores = Q.K^T / sqrt(d) (+ additive mask), Softmax, P.V,
    residual + LayerNorm(eps 1e-12), FFN with erf GELU, residual + LayerNorm.
    All weights N(0, 0.02).  Inputs: int32 token ids [batch, seq] and a float mask
    [batch, seq] of ones."""
    g = GraphBuilder(seed)
    r = g.rng
    d = hidden // heads
    w = lambda *shape: (r.standard_normal(shape) * 0.02).astype(np.float32)
    eps = 1e-12
    ids = g.placeholder("input_ids", [batch, seq], "DT_INT32")
    mask = g.placeholder("attention_mask", [batch, seq])
    emb = g.gather(g.const(w(vocab, hidden)), ids)
    pos = g.const(w(max_pos, hidden)[:seq].reshape(1, seq, hidden))
    x = g.binary("AddV2", emb, pos)
    x = g.layer_norm(x, np.ones(hidden, np.float32) + w(hidden), w(hidden), eps)
    # additive mask: (1 - mask) * -10000, broadcast over heads and query positions
    m = g.reshape(mask, [batch, 1, 1, seq])
    m = g.binary("Mul", g.binary("Sub", g.const(np.float32(1.0)), m), g.const(np.float32(-10000.0)))
    x = g.reshape(x, [batch * seq, hidden])
    for _ in range(layers):
        def heads_of(t):
            t = g.reshape(t, [batch, seq, heads, d])
            return g.transpose(t, [0, 2, 1, 3])
        q = heads_of(g.dense(x, w(hidden, hidden), w(hidden)))
        k = heads_of(g.dense(x, w(hidden, hidden), w(hidden)))
        v = heads_of(g.dense(x, w(hidden, hidden), w(hidden)))
        s = g.batch_matmul(q, k, False, True)
        s = g.binary("Mul", s, g.const(np.float32(1.0 / np.sqrt(d))))
        s = g.binary("AddV2", s, m)
        p = g.node("Softmax", [s], {"T": {"type": "DT_FLOAT"}})
        c = g.batch_matmul(p, v)
        c = g.reshape(g.transpose(c, [0, 2, 1, 3]), [batch * seq, hidden])
        a = g.dense(c, w(hidden, hidden), w(hidden))
        x = g.layer_norm(g.binary("AddV2", x, a), np.ones(hidden, np.float32) + w(hidden),
                         w(hidden), eps)
        h = g.dense(x, w(hidden, ffn), w(ffn))
        # gelu(h) = h * 0.5 * (1 + erf(h / sqrt(2)))
        e = g.unary("Erf", g.binary("Mul", h, g.const(np.float32(1.0 / np.sqrt(2.0)))))
        h = g.binary("Mul", g.binary("Mul", h, g.const(np.float32(0.5))),
                     g.binary("AddV2", e, g.const(np.float32(1.0))))
        f = g.dense(h, w(ffn, hidden), w(hidden))
        x = g.layer_norm(g.binary("AddV2", x, f), np.ones(hidden, np.float32) + w(hidden),
                         w(hidden), eps)
    out = g.reshape(x, [batch, seq, hidden], name="sequence_output")
    return g.artifacts(["input_ids", "attention_mask"], [out])


def flops_per_unit(model, nodes=None):
    """Algorithmic GFLOP per image / sequence of the full-size configurations."""
    return {"mobilenet_v2": 0.601548544, "resnet50": 8.178368512, "bert": 22.347251712}[model]
