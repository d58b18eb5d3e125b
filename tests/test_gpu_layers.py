"""The tfjs-layers way of calling the backend (B200 only): unfused kernel sequences,
LayersModel.predict's slice / execute / concat loop, and what the backend folds behind the
unchanged kernel names.

Checks: the folded launches give the bits of the separate kernels (lazy fusion switched
off) and count fewer launches; MobileNetV2 built the layers way gives the bits of the
converted GraphModel on the same weights and matches the oracle; an encoder block built
from Dense / LayerNormalization / gelu pieces matches a CPU restatement made of the
oracle's kernels within the per-model bounds.
"""
import math

import numpy as np
import pytest

from oracle import graph_oracle, oracle as orc
from tfjs_b200 import layers, model_zoo
from tfjs_b200.graph_model import GraphModel

pytestmark = pytest.mark.gpu


def _both_ways(engine, build, run):
    """run(model) with and without deferred launches: (outputs, launches) per mode."""
    be = engine.backend
    res = {}
    for lazy in (True, False):
        be.lazy_fusion = lazy
        try:
            model = build()
            n0 = be.launch_count()
            out = run(model)
            val = out.arraySync()
            res[lazy] = (val, be.launch_count() - n0)
            out.dispose()
            model.dispose()
        finally:
            be.lazy_fusion = True
    return res


def test_depthwise_bias_relu_clip_is_one_launch_with_the_same_bits(cuda_engine):
    from tfjs_b200 import ops as tf
    r = np.random.default_rng(3)
    x = tf.tensor(r.standard_normal((4, 28, 28, 96)).astype(np.float32))
    kernel = (r.standard_normal((3, 3, 96, 1)) / 3).astype(np.float32)
    bias = r.standard_normal(96).astype(np.float32)
    for act_layer in ("relu_clip", "relu6_activation", "relu", "none"):
        def build():
            dw = layers.DepthwiseConv2D("dw", kernel, bias, 1, "same",
                                        "relu6" if act_layer == "relu6_activation" else
                                        "relu" if act_layer == "relu" else "linear")
            nodes = [(dw, ["input"], "y")]
            if act_layer == "relu_clip":
                nodes.append((layers.ReLU("r", 6.0), ["y"], "z"))
            return layers.LayersModel(["input"], nodes, [nodes[-1][2]])
        res = _both_ways(cuda_engine, build, lambda m: m.predict_on_batch(x))
        assert np.array_equal(res[True][0].view(np.uint32), res[False][0].view(np.uint32)), act_layer
        assert res[True][1] == 1, (act_layer, res[True][1])          # one launch
        assert res[False][1] >= (4 if act_layer.startswith("relu") and act_layer != "relu" else 2)
        ref = orc.fused_depthwise_conv2d(
            x.arraySync(), kernel, 1, "same", bias=bias,
            activation={"none": "linear", "relu": "relu"}.get(act_layer, "relu6"))
        assert np.max(np.abs(res[True][0] - ref)) <= 1e-5 * np.max(np.abs(ref))
    x.dispose()


def test_conv_relu_clip_folds_into_the_convolution(cuda_engine):
    from tfjs_b200 import ops as tf
    r = np.random.default_rng(4)
    x = tf.tensor(r.standard_normal((2, 14, 14, 64)).astype(np.float32))
    kernel = (r.standard_normal((1, 1, 64, 128)) / 8).astype(np.float32)
    bias = r.standard_normal(128).astype(np.float32)

    def build():
        return layers.LayersModel(["input"], [
            (layers.Conv2D("c", kernel, bias, 1, "same", "linear"), ["input"], "y"),
            (layers.ReLU("r", 6.0), ["y"], "z")], ["z"])
    res = _both_ways(cuda_engine, build, lambda m: m.predict_on_batch(x))
    assert np.array_equal(res[True][0].view(np.uint32), res[False][0].view(np.uint32))
    assert res[True][1] == 2 and res[False][1] == 4      # weight packing + 1, against + 3
    x.dispose()


def test_layer_normalization_layers_form(cuda_engine):
    """moments + tile + batchNorm: the tiles are never materialised, the result has the bits
    of the fully materialised sequence, and matches the oracle's kernels."""
    from tfjs_b200 import ops as tf
    r = np.random.default_rng(5)
    for shape in ((6, 128, 768), (33, 100), (2, 3, 5, 64)):
        xv = (r.standard_normal(shape) * 2 + 0.3).astype(np.float32)
        gamma = (1 + r.standard_normal(shape[-1]) * 0.1).astype(np.float32)
        beta = r.standard_normal(shape[-1]).astype(np.float32)
        x = tf.tensor(xv)

        def build():
            return layers.LayersModel(["input"], [
                (layers.LayerNormalization("ln", gamma, beta, 1e-5), ["input"], "y")], ["y"])
        res = _both_ways(cuda_engine, build, lambda m: m.predict_on_batch(x))
        assert np.array_equal(res[True][0].view(np.uint32), res[False][0].view(np.uint32)), shape
        assert res[True][1] == 5 and res[False][1] == 9, (shape, res[True][1], res[False][1])
        mean = orc.reduce("mean", xv, [-1], True)
        var = orc.reduce("mean", orc.unary("square", orc.binary("sub", xv, mean)), [-1], True)
        ref = orc.batch_norm(xv, np.tile(mean, [1] * (len(shape) - 1) + [shape[-1]]),
                             np.tile(var, [1] * (len(shape) - 1) + [shape[-1]]),
                             np.tile(beta.reshape([1] * (len(shape) - 1) + [-1]), list(shape[:-1]) + [1]),
                             np.tile(gamma.reshape([1] * (len(shape) - 1) + [-1]), list(shape[:-1]) + [1]),
                             1e-5)
        assert np.max(np.abs(res[True][0] - ref)) <= 3e-6 * np.max(np.abs(ref)), shape
        x.dispose()


def test_gelu_activation_layers_form_is_one_pass(cuda_engine):
    from tfjs_b200 import ops as tf
    r = np.random.default_rng(6)
    xv = (r.standard_normal((512, 3072)) * 2).astype(np.float32)
    x = tf.tensor(xv)

    def build():
        return layers.LayersModel(["input"], [(layers.Activation("g", "gelu"), ["input"], "y")],
                                  ["y"])
    res = _both_ways(cuda_engine, build, lambda m: m.predict_on_batch(x))
    assert np.array_equal(res[True][0].view(np.uint32), res[False][0].view(np.uint32))
    assert res[True][1] == 1 and res[False][1] == 5
    c = np.float32(math.sqrt(2.0))
    cdf = orc.binary("mul", np.float32(0.5), orc.binary("add", np.float32(1.0),
                                                          orc.unary("erf", orc.binary("div", xv, c))))
    ref = orc.binary("mul", xv, cdf)
    assert np.max(np.abs(res[True][0] - ref)) <= 1e-6 * np.max(np.abs(ref))
    x.dispose()


def test_mobilenet_v2_layers_predict_matches_graph_model_and_oracle(cuda_engine):
    """predict() in batches of 2 over 5 images (a ragged last batch), against the converted
    GraphModel holding the same weights (same bits: the folded launches are the graph's fused
    kernels) and the oracle."""
    size, batch = 96, 5
    lm = layers.mobilenet_v2(size=size)
    x = np.random.default_rng(8).uniform(-1, 1, (batch, size, size, 3)).astype(np.float32)
    xt = cuda_engine.make_tensor(x)
    be = cuda_engine.backend
    before = be.numDataIds()
    y = lm.predict(xt, batch_size=2)
    got = y.arraySync()
    y.dispose()
    assert be.numDataIds() == before            # nothing leaked by the loop
    model_json, weights = model_zoo.mobilenet_v2(batch, size=size)
    gm = GraphModel(model_json, weights, cuda_engine, replay=False)
    # a batch of 2 and a batch of 5 may pick different GEMM tile schedules: TF32 noise bound
    z = gm.execute(xt)
    want = z.arraySync()
    z.dispose()
    assert np.max(np.abs(got - want)) <= 2e-3 * np.max(np.abs(want))
    one = lm.predict(xt, batch_size=batch)       # the same batch size: the same kernels
    same = one.arraySync()
    one.dispose()
    assert np.array_equal(same.view(np.uint32), want.view(np.uint32))
    ref = graph_oracle.run(model_json, weights, {"input": x})["logits"]
    assert np.max(np.abs(got - ref)) <= 1e-2 * np.max(np.abs(ref))
    assert np.array_equal(got.argmax(-1), ref.argmax(-1))
    for t in (xt,):
        t.dispose()
    gm.dispose()
    lm.dispose()


def _oracle_encoder(lm, x, mask, seq, hidden, heads, eps):
    """The encoder stack of layers.bert_encoder restated with the oracle's kernels, reading
    the weights back from the layers."""
    d = hidden // heads
    w = lambda layer, key: layer.weights[key].arraySync()
    dense = lambda layer, v, act="linear": orc.fused_matmul(
        v.reshape(-1, v.shape[-1]), w(layer, "kernel"), False, False, bias=w(layer, "bias"),
        activation=act).reshape(list(v.shape[:-1]) + [-1])

    def layer_norm(layer, v):
        mean = orc.reduce("mean", v, [-1], True)
        var = orc.reduce("mean", orc.unary("square", orc.binary("sub", v, mean)), [-1], True)
        tile = lambda t: np.ascontiguousarray(np.broadcast_to(t, v.shape))
        return orc.batch_norm(v, tile(mean), tile(var), tile(w(layer, "beta")),
                              tile(w(layer, "gamma")), eps)

    def gelu(v):
        c = np.float32(math.sqrt(2.0))
        cdf = orc.binary("mul", np.float32(0.5), orc.binary(
            "add", np.float32(1.0), orc.unary("erf", orc.binary("div", v, c))))
        return orc.binary("mul", v, cdf)
    ls = [n[0] for n in lm.nodes]
    for base in range(0, len(ls), 11):
        q, k, v, _, o, _, ln1, f1, f2, _, ln2 = ls[base:base + 11]
        split = lambda t: orc.transpose(t.reshape(t.shape[0], seq, heads, d), [0, 2, 1, 3])
        qh, kh, vh = split(dense(q, x)), split(dense(k, x)), split(dense(v, x))
        s = orc.batch_matmul(qh, kh, False, True)
        s = orc.binary("add", orc.binary("mul", s, np.float32(1.0 / math.sqrt(d))), mask)
        c = orc.batch_matmul(orc.softmax(s), vh)
        c = orc.transpose(c, [0, 2, 1, 3]).reshape(c.shape[0], seq, hidden)
        x1 = layer_norm(ln1, orc.binary("add", x, dense(o, c)))
        h = gelu(dense(f1, x1))
        x = layer_norm(ln2, orc.binary("add", x1, dense(f2, h)))
    return x


def test_encoder_block_layers_way_matches_oracle(cuda_engine):
    seq, hidden, heads, ffn, batch = 64, 256, 4, 1024, 3
    lm = layers.bert_encoder(seq=seq, layers=2, hidden=hidden, heads=heads, ffn=ffn, seed=2)
    r = np.random.default_rng(9)
    x = r.standard_normal((batch, seq, hidden)).astype(np.float32)
    mask = np.zeros((batch, 1, 1, seq), np.float32)
    mask[1, 0, 0, 50:] = -10000.0
    xt, mt = cuda_engine.make_tensor(x), cuda_engine.make_tensor(mask)
    be = cuda_engine.backend
    outs = {}
    for lazy in (True, False):
        be.lazy_fusion = lazy
        try:
            n0 = be.launch_count()
            y = lm.predict([xt, mt], batch_size=2)
            outs[lazy] = (y.arraySync(), be.launch_count() - n0)
            y.dispose()
        finally:
            be.lazy_fusion = True
    assert np.array_equal(outs[True][0].view(np.uint32), outs[False][0].view(np.uint32))
    assert outs[True][1] < outs[False][1]
    ref = _oracle_encoder(lm, x, mask, seq, hidden, heads, 1e-12)
    assert np.max(np.abs(outs[True][0] - ref)) <= 1e-2 * np.max(np.abs(ref))
    for t in (xt, mt):
        t.dispose()
    lm.dispose()
