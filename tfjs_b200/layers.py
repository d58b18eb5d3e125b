"""The op sequences tfjs-layers issues, for driving the 'cuda' backend the LayersModel way.

In a Node deployment the unmodified tfjs-layers package plays this role; this module
reproduces what its layers call, kernel by kernel, so the same kernel funcs, registered
under the same names, can be exercised and timed from Python:

  LayersModel.predict -> predictLoop: batches of `batchSize` sliced along axis 0, one
      execute per batch, results concatenated (tfjs-layers/src/engine/training.ts:1033-1080,
      backend/tfjs_backend.ts:150-180)
  Conv2D      fused.conv2d with the bias and, for relu / linear / elu only, the activation
              fused; other activations applied afterwards (layers/convolutional.ts:561-600,
              utils/generic_utils.ts:510-522)
  DepthwiseConv2D  depthwiseConv2d, then Add with the bias reshaped to [1, 1, 1, C], then
              the activation (layers/convolutional_depthwise.ts:154-169)
  Dense       fused.matMul for relu / linear / elu, else matMul + biasAdd + activation
              (layers/core.ts:265-290)
  ReLU        relu, then clipByValue(0, maxValue) (layers/advanced_activations.ts)
  relu6 / gelu activations  minimum(6, relu(x));  x * (0.5 * (1 + erf(x / sqrt 2)))
              (activations.ts:83-89, :223-233)
  LayerNormalization  moments, the moments and gamma / beta tiled to the input's shape,
              batchNorm on the tiles (layers/normalization.ts:578-622)
  BatchNormalization (inference)  batchNorm with the moving statistics
              (layers/normalization.ts:44-70)

How the backend answers these sequences (a depthwise convolution whose bias Add, Relu and
clip join its launch; tiles that are never materialised; the gelu chain as one pass) is its
own business: every kernel func keeps the reference's results.
"""
import math

import numpy as np

from . import ops

FUSABLE = ("relu", "linear", "elu")      # mapActivationToFusedKernel


def _dispose(tensors):
    for t in tensors:
        if t is not None and not t.isDisposed:
            t.dispose()


def apply_activation(name, x):
    """activations.ts: the ops an Activation.apply issues.  Returns a new tensor (or x
    itself for 'linear')."""
    if name in (None, "linear"):
        return x
    if name == "relu":
        return ops.relu(x)
    if name == "relu6":
        r = ops.relu(x)
        six = ops.tensor(np.float32(6.0))
        try:
            return ops.minimum(six, r)
        finally:
            _dispose([r, six])
    if name == "gelu":
        c = ops.tensor(np.float32(math.sqrt(2.0)))
        one, half = ops.tensor(np.float32(1.0)), ops.tensor(np.float32(0.5))
        d = ops.div(x, c)
        e = ops.erf(d)
        s = ops.add(one, e)
        cdf = ops.mul(half, s)
        try:
            return ops.mul(x, cdf)
        finally:
            _dispose([c, one, half, d, e, s, cdf])
    if name == "softmax":
        return ops.softmax(x)
    if name == "sigmoid":
        return ops.sigmoid(x)
    if name == "tanh":
        return ops.tanh(x)
    if name == "elu":
        return ops.elu(x)
    raise ValueError("Unknown activation: %s" % name)


class Layer(object):
    """A layer owns its weights as tensors of the active backend and maps input tensors to
    a new output tensor; it never disposes its inputs."""

    def __init__(self, name):
        self.name = name
        self.weights = {}

    def add_weight(self, key, values):
        if values is None:
            return None
        self.weights[key] = ops.tensor(np.asarray(values))
        return self.weights[key]

    def dispose(self):
        _dispose(self.weights.values())
        self.weights = {}


class Conv2D(Layer):
    def __init__(self, name, kernel, bias=None, strides=1, padding="same", activation="linear"):
        super().__init__(name)
        self.kernel, self.bias = self.add_weight("kernel", kernel), self.add_weight("bias", bias)
        self.strides, self.padding, self.activation = strides, padding, activation or "linear"

    def call(self, x):
        fused = self.activation if self.activation in FUSABLE else None
        y = ops.fused_conv2d(x, self.kernel, self.strides, self.padding, "NHWC", [1, 1], None,
                             self.bias, fused or "linear")
        if fused is not None:
            return y
        try:
            return apply_activation(self.activation, y)
        finally:
            _dispose([y])


class DepthwiseConv2D(Layer):
    def __init__(self, name, kernel, bias=None, strides=1, padding="same", activation="linear"):
        super().__init__(name)
        self.kernel, self.bias = self.add_weight("kernel", kernel), self.add_weight("bias", bias)
        self.strides, self.padding, self.activation = strides, padding, activation or "linear"

    def call(self, x):
        tmp = []
        y = ops.depthwise_conv2d(x, self.kernel, self.strides, self.padding, "NHWC", [1, 1])
        if self.bias is not None:
            b4 = ops.reshape(self.bias, [1, 1, 1, self.bias.shape[0]])     # K.biasAdd
            tmp += [y, b4]
            y = ops.add(y, b4)
        out = apply_activation(self.activation, y)
        if out is not y:
            tmp.append(y)
        _dispose(tmp)
        return out


class Dense(Layer):
    def __init__(self, name, kernel, bias=None, activation="linear"):
        super().__init__(name)
        self.kernel, self.bias = self.add_weight("kernel", kernel), self.add_weight("bias", bias)
        self.activation = activation or "linear"

    def call(self, x):
        # K.dot (backend/tfjs_backend.ts:389-450): inputs of rank > 2 are flattened to
        # [-1, lastDim] around the product
        tmp = []
        x2 = x
        if len(x.shape) > 2:
            x2 = ops.reshape(x, [-1, x.shape[-1]])
            tmp.append(x2)
        if self.activation in FUSABLE:
            y = ops.fused_mat_mul(x2, self.kernel, False, False, self.bias, self.activation)
        else:
            y = ops.mat_mul(x2, self.kernel)
        if len(x.shape) > 2:
            tmp.append(y)
            y = ops.reshape(y, list(x.shape[:-1]) + [self.kernel.shape[1]])
        if self.activation in FUSABLE:
            _dispose(tmp)
            return y
        if self.bias is not None:
            tmp.append(y)
            y = ops.add(y, self.bias)                         # K.biasAdd
        out = apply_activation(self.activation, y)
        if out is not y:
            tmp.append(y)
        _dispose(tmp)
        return out


class ReLU(Layer):
    def __init__(self, name, max_value=None):
        super().__init__(name)
        self.max_value = max_value

    def call(self, x):
        y = ops.relu(x)
        if self.max_value is None:
            return y
        try:
            return ops.clip_by_value(y, 0, self.max_value)
        finally:
            _dispose([y])


class Activation(Layer):
    def __init__(self, name, activation):
        super().__init__(name)
        self.activation = activation

    def call(self, x):
        out = apply_activation(self.activation, x)
        return ops.identity(x) if out is x else out


class Add(Layer):
    """Merge layer: tfc.add over the inputs, left to right (layers/merge.ts)."""

    def call(self, *xs):
        out = ops.add(xs[0], xs[1])
        for x in xs[2:]:
            nxt = ops.add(out, x)
            out.dispose()
            out = nxt
        return out


class GlobalAveragePooling2D(Layer):
    def call(self, x):
        return ops.mean(x, [1, 2])


class Reshape(Layer):
    def __init__(self, name, target_shape):
        super().__init__(name)
        self.target_shape = list(target_shape)

    def call(self, x):
        return ops.reshape(x, [x.shape[0]] + self.target_shape)


class Permute(Layer):
    def __init__(self, name, dims):
        super().__init__(name)
        self.dims = list(dims)          # 1-based, the batch axis stays first

    def call(self, x):
        return ops.transpose(x, [0] + self.dims)


class Embedding(Layer):
    def __init__(self, name, embeddings):
        super().__init__(name)
        self.embeddings = self.add_weight("embeddings", embeddings)

    def call(self, ids):
        idx = ids if ids.dtype == "int32" else ops.cast(ids, "int32")
        try:
            flat = ops.reshape(idx, [idx.size])
            out = ops.gather(self.embeddings, flat, 0)
            try:
                return ops.reshape(out, list(ids.shape) + [self.embeddings.shape[1]])
            finally:
                _dispose([flat, out])
        finally:
            if idx is not ids:
                idx.dispose()


class LayerNormalization(Layer):
    """layers/normalization.ts:578-622 for axis = -1."""

    def __init__(self, name, gamma, beta, epsilon=1e-3):
        super().__init__(name)
        self.gamma, self.beta = self.add_weight("gamma", gamma), self.add_weight("beta", beta)
        self.epsilon = epsilon

    def call(self, x):
        rank = len(x.shape)
        tmp = []
        keep = lambda t: (tmp.append(t), t)[1]
        try:
            # tfc.moments(x, [-1], keepDims = true)
            mean = keep(ops.mean(x, [rank - 1], True))
            dev = keep(ops.sub(x, mean))
            sq = keep(ops.square(dev))
            variance = keep(ops.mean(sq, [rank - 1], True))
            bshape = [1] * (rank - 1) + [x.shape[-1]]
            scale = keep(ops.reshape(self.gamma, bshape)) if self.gamma is not None else None
            offset = keep(ops.reshape(self.beta, bshape)) if self.beta is not None else None
            moments_tiling = [1] * (rank - 1) + [x.shape[-1]]
            scale_tiling = list(x.shape[:-1]) + [1]
            mean_t = keep(ops.tile(mean, moments_tiling))
            var_t = keep(ops.tile(variance, moments_tiling))
            scale_t = keep(ops.tile(scale, scale_tiling)) if scale is not None else None
            offset_t = keep(ops.tile(offset, scale_tiling)) if offset is not None else None
            return ops.batch_norm(x, mean_t, var_t, offset_t, scale_t, self.epsilon)
        finally:
            _dispose(tmp)


class BatchNormalization(Layer):
    """Inference form: batchNorm with the moving statistics over the last axis."""

    def __init__(self, name, gamma, beta, moving_mean, moving_variance, epsilon=1e-3):
        super().__init__(name)
        self.gamma, self.beta = self.add_weight("gamma", gamma), self.add_weight("beta", beta)
        self.mean = self.add_weight("moving_mean", moving_mean)
        self.variance = self.add_weight("moving_variance", moving_variance)
        self.epsilon = epsilon

    def call(self, x):
        return ops.batch_norm(x, self.mean, self.variance, self.beta, self.gamma, self.epsilon)


class Lambda(Layer):
    """A layer whose call is given as a function of the ops module and the inputs (the
    attention arithmetic of the encoder block below; tfjs-layers users write such blocks
    with tf.* ops inside a custom layer's call)."""

    def __init__(self, name, fn):
        super().__init__(name)
        self.fn = fn

    def call(self, *xs):
        return self.fn(ops, *xs)


class LayersModel(object):
    """A functional model: `nodes` is a topologically ordered list of
    (layer, [input names], output name); `inputs` / `outputs` name the feeds and results."""

    def __init__(self, inputs, nodes, outputs):
        self.inputs, self.nodes, self.outputs = list(inputs), list(nodes), list(outputs)
        last_use = {}
        for pos, (_, ins, _) in enumerate(self.nodes):
            for name in ins:
                last_use[name] = pos
        self._last_use = last_use

    def predict_on_batch(self, xs):
        """One execute of the layer graph (training.ts execute()): intermediate tensors are
        disposed after their last consumer, like the tidy() scopes of the reference."""
        xs = xs if isinstance(xs, (list, tuple)) else [xs]
        values = dict(zip(self.inputs, xs))
        owned = set()
        try:
            for pos, (layer, ins, out) in enumerate(self.nodes):
                values[out] = layer.call(*[values[n] for n in ins])
                owned.add(out)
                for n in ins:
                    if n in owned and self._last_use[n] == pos and n not in self.outputs:
                        values[n].dispose()
                        owned.discard(n)
        except Exception:
            _dispose(values[n] for n in owned)
            raise
        _dispose(values[n] for n in owned if n not in self.outputs)
        res = [values[n] for n in self.outputs]
        return res if len(res) > 1 else res[0]

    def predict(self, xs, batch_size=32):
        """LayersModel.predict -> predictLoop (training.ts:1033-1080)."""
        xs = xs if isinstance(xs, (list, tuple)) else [xs]
        num = xs[0].shape[0]
        outs = [[] for _ in self.outputs]
        for start in range(0, num, batch_size):
            size = min(batch_size, num - start)
            batch = [ops.slice(x, [start] + [0] * (len(x.shape) - 1), [size] + list(x.shape[1:]))
                     for x in xs]                       # sliceAlongFirstAxis
            res = self.predict_on_batch(batch)
            _dispose(batch)
            for i, t in enumerate(res if isinstance(res, list) else [res]):
                outs[i].append(t)
        merged = []
        for parts in outs:
            merged.append(ops.concat(parts, 0))
            _dispose(parts)
        return merged if len(merged) > 1 else merged[0]

    def dispose(self):
        for layer, _, _ in self.nodes:
            layer.dispose()


# ------------------------------------------------------------------ model builders --
def mobilenet_v2(size=224, classes=1000, seed=0):
    """MobileNetV2-1.0 as Keras / tfjs-layers builds it, with the weights of
    model_zoo.mobilenet_v2 (BatchNorm folded into the convolution biases): Conv2D(linear)
    -> ReLU(6) for the expand and stem convolutions, DepthwiseConv2D(+bias) -> ReLU(6),
    Conv2D(linear) projection, Add for the residual blocks."""
    from . import model_zoo
    r = np.random.default_rng(seed)
    bias = lambda c: (r.standard_normal(c) * 0.01).astype(np.float32)
    nodes, n = [], [0]

    def add(layer_cls, ins, *args, **kw):
        n[0] += 1
        out = "t%d" % n[0]
        nodes.append((layer_cls("l%d" % n[0], *args, **kw), ins, out))
        return out
    x = "input"
    c_in = 32
    x = add(Conv2D, [x], model_zoo._glorot(r, (3, 3, 3, c_in), 27, 9 * c_in), bias(c_in), 2, "same")
    x = add(ReLU, [x], 6.0)
    for t, c, reps, s in ((1, 16, 1, 1), (6, 24, 2, 2), (6, 32, 3, 2), (6, 64, 4, 2),
                          (6, 96, 3, 1), (6, 160, 3, 2), (6, 320, 1, 1)):
        for i in range(reps):
            stride = s if i == 0 else 1
            y, c_mid = x, c_in * t
            if t != 1:
                y = add(Conv2D, [y], model_zoo._glorot(r, (1, 1, c_in, c_mid), c_in, c_mid),
                        bias(c_mid), 1, "same")
                y = add(ReLU, [y], 6.0)
            y = add(DepthwiseConv2D, [y], model_zoo._glorot(r, (3, 3, c_mid, 1), 9, 9), bias(c_mid),
                    stride, "same")
            y = add(ReLU, [y], 6.0)
            y = add(Conv2D, [y], model_zoo._glorot(r, (1, 1, c_mid, c), c_mid, c), bias(c), 1,
                    "same")
            if stride == 1 and c_in == c:
                y = add(Add, [x, y])
            x, c_in = y, c
    x = add(Conv2D, [x], model_zoo._glorot(r, (1, 1, c_in, 1280), c_in, 1280), bias(1280), 1, "same")
    x = add(ReLU, [x], 6.0)
    x = add(GlobalAveragePooling2D, [x])
    x = add(Dense, [x], model_zoo._glorot(r, (1280, classes), 1280, classes), bias(classes))
    return LayersModel(["input"], nodes, [x])


def encoder_block(x_name, nodes, counter, r, seq, hidden, heads, ffn, eps):
    """One post-LayerNorm transformer encoder layer written with tfjs-layers pieces: Dense
    projections, a custom attention layer, Add, LayerNormalization, Dense(gelu)."""
    d = hidden // heads
    w = lambda *shape: (r.standard_normal(shape) * 0.02).astype(np.float32)

    def add(layer_cls, ins, *args, **kw):
        counter[0] += 1
        out = "t%d" % counter[0]
        nodes.append((layer_cls("l%d" % counter[0], *args, **kw), ins, out))
        return out

    def split_heads(tf, t):
        b = t.shape[0]
        r4 = tf.reshape(t, [b, seq, heads, d])
        try:
            return tf.transpose(r4, [0, 2, 1, 3])
        finally:
            r4.dispose()

    def attention(tf, q, k, v, mask):
        qh, kh, vh = split_heads(tf, q), split_heads(tf, k), split_heads(tf, v)
        scale = tf.tensor(np.float32(1.0 / math.sqrt(d)))
        s = tf.mat_mul(qh, kh, False, True)
        s2 = tf.mul(s, scale)
        s3 = tf.add(s2, mask)
        p = tf.softmax(s3)
        c = tf.mat_mul(p, vh)
        ct = tf.transpose(c, [0, 2, 1, 3])
        try:
            return tf.reshape(ct, [ct.shape[0], seq, hidden])
        finally:
            for t in (qh, kh, vh, scale, s, s2, s3, p, c, ct):
                t.dispose()
    q = add(Dense, [x_name], w(hidden, hidden), w(hidden))
    k = add(Dense, [x_name], w(hidden, hidden), w(hidden))
    v = add(Dense, [x_name], w(hidden, hidden), w(hidden))
    a = add(Lambda, [q, k, v, "mask"], attention)
    a = add(Dense, [a], w(hidden, hidden), w(hidden))
    x1 = add(Add, [x_name, a])
    x1 = add(LayerNormalization, [x1], np.ones(hidden, np.float32) + w(hidden), w(hidden), eps)
    h = add(Dense, [x1], w(hidden, ffn), w(ffn), "gelu")
    f = add(Dense, [h], w(ffn, hidden), w(hidden))
    x2 = add(Add, [x1, f])
    return add(LayerNormalization, [x2], np.ones(hidden, np.float32) + w(hidden), w(hidden), eps)


def bert_encoder(seq=128, layers=12, hidden=768, heads=12, ffn=3072, seed=0, eps=1e-12):
    """A BERT-shaped encoder stack over already embedded inputs: feeds are `hidden_in`
    [batch, seq, hidden] and the additive attention `mask` [batch, 1, 1, seq]."""
    r = np.random.default_rng(seed)
    nodes, counter = [], [0]
    x = "hidden_in"
    for _ in range(layers):
        x = encoder_block(x, nodes, counter, r, seq, hidden, heads, ffn, eps)
    return LayersModel(["hidden_in", "mask"], nodes, [x])
