"""Graph models on the CUDA backend vs the CPU oracle (B200 only).

Two checks per model, on the same seeded inputs:
  (a) per layer: every node is run on the GPU with the ORACLE's inputs for that
      node, so only that kernel's own error shows; bound max|err| <= 2e-3 * max|ref|
      (TF32 operands, fp32 accumulation).
  (b) end to end: one GPU forward pass, every node output compared with the
      oracle's; TF32 rounding noise accumulates over ~50 layers as a random walk,
      so the bound here is 1e-2 * max|ref| per node, and the final arg-max must be
      identical.
Batches are small so that the scalar oracle finishes in seconds; the layer shapes
per image are the full-size ones.
"""
import numpy as np
import pytest

from oracle import graph_oracle
from tfjs_b200 import model_zoo
from tfjs_b200.graph_model import GraphModel

pytestmark = pytest.mark.gpu
TOL = 2e-3          # per layer, oracle inputs
DRIFT_TOL = 1e-2    # end to end


def _per_layer(engine, model_json, weights, feeds):
    """Check (a): each compute node on the GPU with the oracle's input values."""
    from tfjs_b200 import graph_model
    ref = graph_oracle.run(model_json, weights, feeds)
    gm = GraphModel(model_json, weights, engine)
    worst = ("", 0.0)
    for d in model_json["modelTopology"]["node"]:
        if d["op"] in ("Const", "Placeholder"):
            continue
        node = graph_model.Node(d)
        made, ins = [], []
        for i in node.inputs:
            src = i.split(":")[0]
            if src in gm.weights:
                ins.append(gm.weights[src])
            else:
                v = ref[src]
                t = engine.make_tensor(v, list(v.shape),
                                       "int32" if v.dtype == np.int32 else "float32")
                made.append(t)
                ins.append(t)
        out = graph_model.execute_op(node, ins)
        g = out.arraySync()
        out.dispose()
        for t in made:
            t.dispose()
        r = ref[node.name]
        assert list(g.shape) == list(r.shape), node.name
        denom = float(np.max(np.abs(r))) or 1.0
        err = float(np.max(np.abs(g.astype(np.float64) - r))) / denom
        if err > worst[1]:
            worst = (node.name + ":" + node.op, err)
    gm.dispose()
    return worst


def _run_and_compare(engine, model_json, weights, feeds, out_name, check_nodes=True):
    ref = graph_oracle.run(model_json, weights, feeds)
    gm = GraphModel(model_json, weights, engine)
    gm.executor.keep_intermediates = True
    tensors = {k: engine.make_tensor(v, list(v.shape), "int32" if v.dtype == np.int32 else "float32")
               for k, v in feeds.items()}
    out = gm.execute(tensors, [out_name])[0]
    got = out.arraySync()
    worst = ("", 0.0)
    if check_nodes:
        for name, t in gm.executor.intermediates.items():
            r = ref[name]
            g = t.arraySync()
            assert list(g.shape) == list(r.shape), name
            denom = float(np.max(np.abs(r))) or 1.0
            err = float(np.max(np.abs(g.astype(np.float64) - r))) / denom
            if err > worst[1]:
                worst = (name, err)
    for t in gm.executor.intermediates.values():
        t.dispose()
    for t in tensors.values():
        t.dispose()
    gm.dispose()
    return got, ref[out_name], worst


def test_mobilenet_v2_b2(cuda_engine):
    model_json, weights = model_zoo.mobilenet_v2(2)
    x = np.random.default_rng(1).uniform(-1, 1, (2, 224, 224, 3)).astype(np.float32)
    got, ref, worst = _run_and_compare(cuda_engine, model_json, weights, {"input": x}, "logits")
    assert worst[1] <= DRIFT_TOL, worst
    assert np.array_equal(got.argmax(-1), ref.argmax(-1))
    layer = _per_layer(cuda_engine, model_json, weights, {"input": x})
    assert layer[1] <= TOL, layer


def test_resnet50_uint8_weights_b2(cuda_engine):
    model_json, weights = model_zoo.resnet50(2)
    # weights dequantised on the device are bit-identical to the reference's host loop
    specs = model_json["weightsManifest"][0]["weights"]
    ref_w = graph_oracle.decode_weights(weights, specs)
    gm = GraphModel(model_json, weights, cuda_engine)
    assert any("quantization" in s for s in specs)
    for name in list(ref_w)[:40]:
        assert np.array_equal(gm.weights[name].arraySync(), ref_w[name]), name
    gm.dispose()
    x = np.random.default_rng(2).uniform(0, 1, (2, 224, 224, 3)).astype(np.float32)
    got, ref, worst = _run_and_compare(cuda_engine, model_json, weights, {"input": x}, "logits")
    assert worst[1] <= DRIFT_TOL, worst
    assert np.array_equal(got.argmax(-1), ref.argmax(-1))
    layer = _per_layer(cuda_engine, model_json, weights, {"input": x})
    assert layer[1] <= TOL, layer


def test_bert_encoder_b2(cuda_engine):
    model_json, weights = model_zoo.bert_encoder(2, layers=3)
    r = np.random.default_rng(3)
    feeds = {"input_ids": r.integers(0, 30522, (2, 128)).astype(np.int32),
             "attention_mask": np.ones((2, 128), np.float32)}
    layer = _per_layer(cuda_engine, model_json, weights, feeds)
    assert layer[1] <= TOL, layer
    got, ref, worst = _run_and_compare(cuda_engine, model_json, weights, feeds, "sequence_output",
                                       check_nodes=False)
    denom = float(np.max(np.abs(ref)))
    assert float(np.max(np.abs(got - ref))) / denom <= DRIFT_TOL


def test_no_data_id_leak_across_executes(cuda_engine):
    model_json, weights = model_zoo.mobilenet_v2(1, size=96)
    gm = GraphModel(model_json, weights, cuda_engine)
    x = cuda_engine.make_tensor(np.zeros((1, 96, 96, 3), np.float32))
    base = None
    for _ in range(3):
        y = gm.execute(x)
        y.dataSync()
        y.dispose()
        n = cuda_engine.backend.numDataIds()
        assert base is None or n == base
        base = n
    x.dispose()
    gm.dispose()


# ------------------------------------------------- plan rewrite: layer normalisation --
@pytest.mark.parametrize("mode", ["fp32", "tf32"])
@pytest.mark.parametrize("residual", [None, "same", "broadcast"])
@pytest.mark.parametrize("shape", [(64, 128, 768), (5, 7, 100), (3, 1024), (9, 4), (2, 3, 6),
                                   (4, 2048)])
def test_fused_layer_norm_has_the_bits_of_the_separate_kernels(cuda_engine, shape, residual, mode):
    """One launch against the nine kernels it replaces; shapes the kernel does not take
    (a row that is not a multiple of 4, or beyond 1024) run the separate kernels.  fp32 math
    mode: the same double-precision sums in the same order, bit for bit.  TF32 math mode (the
    default): the one-launch kernel forms its two sums in fp32, within a few units in the
    last place of the separate kernels."""
    from tfjs_b200 import graph_model, ops
    cuda_engine.backend.set_math_mode(mode)
    try:
        got, ref = _layer_norm_both_ways(graph_model, ops, shape, residual)
    finally:
        cuda_engine.backend.set_math_mode("tf32")
    assert got.shape == ref.shape
    if mode == "fp32":
        assert np.array_equal(got.view(np.uint32), ref.view(np.uint32))
    else:
        assert np.max(np.abs(got - ref)) <= 4e-6 * np.max(np.abs(ref))


def _layer_norm_both_ways(graph_model, ops, shape, residual):
    r = np.random.default_rng(sum(shape))
    x = ops.tensor((r.standard_normal(shape) * 3 + 0.5).astype(np.float32))
    extra = []
    if residual is not None:
        rshape = shape if residual == "same" else (1,) + tuple(shape[1:])
        extra = [ops.tensor(r.standard_normal(rshape).astype(np.float32))]
    gamma = ops.tensor(r.standard_normal(shape[-1]).astype(np.float32))
    beta = ops.tensor(r.standard_normal(shape[-1]).astype(np.float32))
    eps = np.float32(1e-12)
    attrs = {"epsilon": {"f": float(eps)}}
    if extra:
        attrs["residual"] = {"b": True}
    node = graph_model.Node({"name": "ln", "op": "_FusedLayerNorm",
                             "input": ["x"] + ["r"] * len(extra) + ["g", "b"], "attr": attrs})
    got_t = graph_model.execute_op(node, [x] + extra + [gamma, beta])
    got = got_t.arraySync()
    if extra:
        extra.append(x)
        x = ops.add(x, extra[0])
    mean = ops.mean(x, [-1], True)
    sq = ops.squared_difference(x, mean)
    var = ops.mean(sq, [-1], True)
    e = ops.tensor(eps)
    ve = ops.add(var, e)
    rs = ops.rsqrt(ve)
    sub = ops.sub(x, mean)
    norm = ops.mul(sub, rs)
    ng = ops.mul(norm, gamma)
    ref_t = ops.add(ng, beta)
    ref = ref_t.arraySync()
    for t in [got_t, mean, sq, var, e, ve, rs, sub, norm, ng, ref_t, x, gamma, beta] + extra:
        t.dispose()
    return got, ref


@pytest.mark.parametrize("mode", ["fp32", "tf32"])
def test_bert_with_fused_layer_norms_matches_the_stored_graph(cuda_engine, mode):
    """fp32 math mode: every rewrite keeps the bits of the stored graph (the attention kernel
    declines that mode).  TF32 math mode: the one-launch layer normalisation sums in fp32 and
    the attention kernel sums its softmax in another order: a tolerance."""
    cuda_engine.backend.set_math_mode(mode)
    try:
        outs = _bert_fused_and_stored(cuda_engine)
    finally:
        cuda_engine.backend.set_math_mode("tf32")
    if mode == "fp32":
        assert np.array_equal(outs[0].view(np.uint32), outs[1].view(np.uint32))
    else:
        assert np.max(np.abs(outs[0] - outs[1])) <= 1e-3 * np.max(np.abs(outs[1]))


def _bert_fused_and_stored(cuda_engine):
    model_json, weights = model_zoo.bert_encoder(2, layers=2)
    r = np.random.default_rng(3)
    feeds = {"input_ids": r.integers(0, 30522, (2, 128)).astype(np.int32),
             "attention_mask": np.ones((2, 128), np.float32)}
    outs = []
    be = cuda_engine.backend
    for fuse in (True, False):
        gm = GraphModel(model_json, weights, cuda_engine, replay=False)
        gm.executor.fuse = fuse
        ins = {k: cuda_engine.make_tensor(v, list(v.shape), "int32" if v.dtype == np.int32
                                          else "float32") for k, v in feeds.items()}
        before = be.numDataIds()
        y = gm.execute(ins, ["sequence_output"])[0]
        outs.append(y.arraySync())
        assert gm.executor.fused_subgraphs == (5 if fuse else 0)
        y.dispose()
        assert be.numDataIds() == before
        for t in ins.values():
            t.dispose()
        gm.dispose()
    return outs


# ---------------------------------------------------- plan rewrite: attention heads --
@pytest.mark.parametrize("heads", [(2, 128, 12, 64), (3, 64, 4, 32), (1, 96, 2, 160),
                                   (2, 50, 3, 64), (2, 64, 3, 48)])
def test_matmul_heads_store_has_the_bits_of_matmul_then_transpose(cuda_engine, heads):
    """Split and merge through the permuted store against product + Reshape + Transpose; the
    last two shapes (S or D not a multiple of 32) are declined by the library and take the
    three ops inside the executor."""
    from tfjs_b200 import graph_model, ops
    import base64
    B, S, H, D = heads
    r = np.random.default_rng(B * 1000 + S)
    enc = lambda t: {"s": base64.b64encode(t.encode()).decode()}
    ints = lambda v: {"list": {"i": [str(x) for x in v]}}
    # split: [B*S, K] x [K, H*D] + bias -> [B, H, S, D]
    K = 96
    a = ops.tensor(r.standard_normal((B * S, K)).astype(np.float32))
    w = ops.tensor((r.standard_normal((K, H * D)) / 8).astype(np.float32))
    bias = ops.tensor(r.standard_normal(H * D).astype(np.float32))
    attrs = {"transpose_a": {"b": False}, "transpose_b": {"b": False}, "num_args": {"i": "1"},
             "fused_ops": {"list": {"s": [base64.b64encode(b"BiasAdd").decode()]}},
             "_layout": enc("split"), "_op": enc("_FusedMatMul"), "_dims": ints([B, S, H, D])}
    node = graph_model.Node({"name": "q", "op": "_MatMulHeads", "input": ["a", "w", "b"],
                             "attr": attrs})
    got_t = graph_model.execute_op(node, [a, w, bias])
    y = ops.fused_mat_mul(a, w, False, False, bias, "linear")
    y4 = ops.reshape(y, [B, S, H, D])
    ref_t = ops.transpose(y4, [0, 2, 1, 3])
    got, ref = got_t.arraySync(), ref_t.arraySync()
    assert got.shape == (B, H, S, D)
    assert np.array_equal(got.view(np.uint32), ref.view(np.uint32))
    # merge: [B, H, S, S] x [B, H, S, D] -> [B, S, H, D] -> [B*S, H*D]
    p = ops.tensor(r.random((B, H, S, S)).astype(np.float32))
    attrs = {"adj_x": {"b": False}, "adj_y": {"b": False}, "_layout": enc("merge"),
             "_op": enc("BatchMatMulV2"), "_dims": ints([B * S, H * D])}
    node = graph_model.Node({"name": "c", "op": "_MatMulHeads", "input": ["p", "v"],
                             "attr": attrs})
    got2_t = graph_model.execute_op(node, [p, ref_t])
    c = ops.mat_mul(p, ref_t)
    ct = ops.transpose(c, [0, 2, 1, 3])
    ref2_t = ops.reshape(ct, [B * S, H * D])
    got2, ref2 = got2_t.arraySync(), ref2_t.arraySync()
    assert got2.shape == (B * S, H * D)
    assert np.array_equal(got2.view(np.uint32), ref2.view(np.uint32))
    for t in (a, w, bias, got_t, y, y4, ref_t, p, got2_t, c, ct, ref2_t):
        t.dispose()


def test_bert_with_folded_head_transposes_matches_the_stored_graph(cuda_engine):
    model_json, weights = model_zoo.bert_encoder(2, layers=2)
    r = np.random.default_rng(4)
    feeds = {"input_ids": r.integers(0, 30522, (2, 128)).astype(np.int32),
             "attention_mask": np.ones((2, 128), np.float32)}
    outs, launches = [], []
    be = cuda_engine.backend
    # every rewrite but two keeps the bits of the stored graph in the default math mode: the
    # attention kernel forms the softmax's sum in another order, the one-launch layer
    # normalisation its two sums in fp32
    for fuse, skip in ((True, {"attention", "layernorm"}), (False, set()), (True, set())):
        gm = GraphModel(model_json, weights, cuda_engine, replay=False)
        gm.executor.fuse = fuse
        gm.executor.fuse_skip = set(skip)
        ins = {k: cuda_engine.make_tensor(v, list(v.shape), "int32" if v.dtype == np.int32
                                          else "float32") for k, v in feeds.items()}
        before = be.numDataIds()
        y = gm.execute(ins, ["sequence_output"])[0]
        outs.append(y.arraySync())
        assert gm.executor.fused_heads == (8 if fuse else 0)
        assert gm.executor.fused_softmaxes == (2 if fuse else 0)
        assert gm.executor.fused_gelus == (2 if fuse else 0)
        assert gm.executor.fused_attentions == (2 if fuse and not skip else 0)
        y.dispose()
        assert be.numDataIds() == before
        for t in ins.values():
            t.dispose()
        gm.dispose()
    assert np.array_equal(outs[0].view(np.uint32), outs[1].view(np.uint32))
    assert np.max(np.abs(outs[2] - outs[1])) <= 1e-3 * np.max(np.abs(outs[1]))


# ------------------------------------------------- plan rewrite: softmax of scores --
@pytest.mark.parametrize("case", [((4, 6, 64, 128), (4, 1, 1, 128), 0.125),
                                  ((4, 6, 64, 128), (4, 6, 64, 128), 0.5),
                                  ((3, 5, 40), (40,), 0.3), ((2, 3, 8, 2000), (2, 1, 1, 2000), 2.0),
                                  ((4, 6, 64, 128), None, 0.125),
                                  ((4, 6, 16, 32), (1, 6, 1, 32), 0.125)])
def test_scaled_masked_softmax_has_the_bits_of_the_separate_kernels(cuda_engine, case):
    """The last case's mask does not broadcast over whole rows: the executor runs the three
    kernels."""
    from tfjs_b200 import graph_model, ops
    xs, ms, scale = case
    r = np.random.default_rng(len(xs) * 100 + xs[-1])
    x = ops.tensor((r.standard_normal(xs) * 4).astype(np.float32))
    mask = None if ms is None else ops.tensor(
        np.where(r.random(ms) < 0.2, -10000.0, 0.0).astype(np.float32))
    node = graph_model.Node({"name": "p", "op": "_SoftmaxScaledMasked",
                             "input": ["x"] + (["m"] if ms else []),
                             "attr": {"_scale": {"f": float(np.float32(scale))}}})
    got_t = graph_model.execute_op(node, [x] + ([mask] if ms else []))
    c = ops.tensor(np.float32(scale))
    s1 = ops.mul(x, c)
    s2 = ops.add(s1, mask) if ms else ops.identity(s1)
    ref_t = ops.softmax(s2)
    got, ref = got_t.arraySync(), ref_t.arraySync()
    for t in [x, got_t, c, s1, s2, ref_t] + ([mask] if ms else []):
        t.dispose()
    assert np.array_equal(got.view(np.uint32), ref.view(np.uint32))


# ------------------------------------------------------ plan rewrite: erf GELU --
@pytest.mark.parametrize("mode", ["tf32", "fp32"])
@pytest.mark.parametrize("divide", [False, True])
def test_gelu_epilogue_has_the_bits_of_the_five_kernels(cuda_engine, mode, divide):
    from tfjs_b200 import graph_model, ops
    import base64
    r = np.random.default_rng(11)
    a = ops.tensor(r.standard_normal((300, 96)).astype(np.float32))
    w = ops.tensor((r.standard_normal((96, 200)) / 4).astype(np.float32))
    bias = ops.tensor(r.standard_normal(200).astype(np.float32))
    c = float(np.float32(np.sqrt(2.0))) if divide else float(np.float32(1 / np.sqrt(2.0)))
    attrs = {"transpose_a": {"b": False}, "transpose_b": {"b": False}, "num_args": {"i": "1"},
             "fused_ops": {"list": {"s": [base64.b64encode(b"BiasAdd").decode()]}},
             "_gelu": {"list": {"f": [c, 0.5, 1.0, 1.0 if divide else 0.0]}}}
    node = graph_model.Node({"name": "h", "op": "_FusedMatMulGelu", "input": ["a", "w", "b"],
                             "attr": attrs})
    cuda_engine.backend.set_math_mode(mode)
    try:
        got_t = graph_model.execute_op(node, [a, w, bias])
        h = ops.fused_mat_mul(a, w, False, False, bias, "linear")
        ct, half, one = ops.tensor(np.float32(c)), ops.tensor(np.float32(0.5)), ops.tensor(np.float32(1))
        s = ops.div(h, ct) if divide else ops.mul(h, ct)
        e = ops.erf(s)
        e1 = ops.add(e, one)
        m = ops.mul(h, half)
        ref_t = ops.mul(m, e1)
        got, ref = got_t.arraySync(), ref_t.arraySync()
    finally:
        cuda_engine.backend.set_math_mode("tf32")
    for t in (a, w, bias, got_t, h, ct, half, one, s, e, e1, m, ref_t):
        t.dispose()
    assert np.array_equal(got.view(np.uint32), ref.view(np.uint32))
