"""Whole-step capture and replay (B200 only).

GraphModel(replay=True) runs a signature eagerly once, captures the second execute
into a CUDA graph and replays it afterwards.  A replay must give the bits of the
eager path for fresh inputs, count its kernels, leave no tensors behind, and a step
that cannot be captured must fall back to eager execution with the context intact.
"""
import ctypes

import numpy as np
import pytest

from tfjs_b200 import model_zoo
from tfjs_b200.graph_model import GraphModel

pytestmark = pytest.mark.gpu


def _feeds(kind, seed):
    r = np.random.default_rng(seed)
    if kind == "bert":
        return {"input_ids": r.integers(0, 30522, (2, 128)).astype(np.int32),
                "attention_mask": np.ones((2, 128), np.float32)}
    return {"input": r.uniform(-1, 1, (2, 96, 96, 3)).astype(np.float32)}


def _model(kind):
    if kind == "mobilenet":
        return model_zoo.mobilenet_v2(2, size=96) + ("logits",)
    if kind == "resnet":
        return model_zoo.resnet50(2, size=96) + ("logits",)
    return model_zoo.bert_encoder(2, layers=2) + ("sequence_output",)


@pytest.mark.parametrize("kind", ["mobilenet", "resnet", "bert"])
def test_replay_matches_eager_bit_for_bit(cuda_engine, kind):
    model_json, weights, out_name = _model(kind)
    eager = GraphModel(model_json, weights, cuda_engine, replay=False)
    fast = GraphModel(model_json, weights, cuda_engine, replay=True)
    be = cuda_engine.backend
    states, per_step = [], []
    for step in range(5):
        feeds = _feeds(kind, 100 + step)
        ins = {k: cuda_engine.make_tensor(v, list(v.shape),
                                          "int32" if v.dtype == np.int32 else "float32")
               for k, v in feeds.items()}
        want = eager.execute(ins, [out_name])[0]
        n0 = be.launch_count()
        got = fast.execute(ins, [out_name])[0]
        per_step.append(be.launch_count() - n0)
        states.append(list(fast._replays.values())[0]["state"])
        a, b = want.dataSync(), got.dataSync()
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32)), (kind, step)
        for t in list(ins.values()) + [want, got]:
            t.dispose()
    assert states == ["warm", "ready", "ready", "ready", "ready"], \
        (states, list(fast._replays.values())[0].get("why"))
    # a replay launches the step's kernels plus the input / output copies' none
    assert per_step[2] == per_step[3] == per_step[4] > 0
    base = cuda_engine.memory()["numTensors"]
    fast.dispose()
    eager.dispose()
    assert cuda_engine.memory()["numTensors"] < base


def test_refused_call_discards_the_capture_and_keeps_the_context(cuda_engine):
    from tfjs_b200 import ops as tf
    be = cuda_engine.backend
    lib = be.lib
    a = tf.tensor(np.arange(1 << 16, dtype=np.float32))
    aid = be.device_id(a.dataId)
    be.capture_begin(1 << 20)
    host = np.zeros(4, np.float32)
    rc = lib.tfjs_cuda_write(be.ctx, aid, host.ctypes.data_as(ctypes.c_void_p), 16)
    assert rc == 5                                     # TFJS_CUDA_UNSUPPORTED
    assert lib.tfjs_cuda_sync(be.ctx) == 5
    graph = ctypes.c_int32(7)
    rc = lib.tfjs_cuda_capture_end(be.ctx, 0, ctypes.byref(graph))
    assert rc == 5 and graph.value == 0
    assert b"captured step" in lib.tfjs_cuda_last_error(be.ctx)
    # the context still works
    b = tf.add(a, a)
    assert np.array_equal(b.dataSync(), 2 * np.arange(1 << 16, dtype=np.float32))
    # arena exhaustion is reported, not a fault
    be.capture_begin(256)
    out = ctypes.c_int32()
    assert lib.tfjs_cuda_alloc(be.ctx, 1 << 20, ctypes.byref(out)) == 2   # OUT_OF_MEMORY
    assert lib.tfjs_cuda_capture_end(be.ctx, 0, ctypes.byref(graph)) == 5
    assert lib.tfjs_cuda_graph_launch(be.ctx, 99) == 4                    # UNKNOWN_ID
    c = tf.relu(b)
    assert np.array_equal(c.dataSync(), 2 * np.arange(1 << 16, dtype=np.float32))
    for t in (a, b, c):
        t.dispose()


def test_uncapturable_model_stays_eager(cuda_engine, monkeypatch):
    """A kernel that has to ask the host in the middle of a step (here: forced by
    making every Relu6 read its input back) makes the capture fail once; execution
    continues eagerly with correct results."""
    from tfjs_b200 import graph_model
    model_json, weights, out_name = _model("mobilenet")
    gm = GraphModel(model_json, weights, cuda_engine, replay=True)
    real = graph_model.execute_op

    def nosy(node, inp):
        out = real(node, inp)
        if node.op == "Mean":
            out.dataSync()            # a device-to-host read inside the step
        return out
    monkeypatch.setattr(graph_model, "execute_op", nosy)
    ref = GraphModel(model_json, weights, cuda_engine, replay=False)
    for step in range(3):
        feeds = _feeds("mobilenet", step)
        ins = {k: cuda_engine.make_tensor(v) for k, v in feeds.items()}
        got = gm.execute(ins, [out_name])[0]
        want = ref.execute(ins, [out_name])[0]
        assert np.array_equal(got.dataSync(), want.dataSync())
        for t in list(ins.values()) + [got, want]:
            t.dispose()
    st = list(gm._replays.values())[0]
    assert st["state"] == "eager" and "captured step" in st["why"]
    gm.dispose()
    ref.dispose()


def _im2col_model(batch, seed=5):
    """One convolution whose channel count (6) and reduction length (11 * 11 * 6 = 726) send
    it down the explicit im2col path, which writes the context's scratch buffer, followed by
    a 3x3 convolution with a packed weight."""
    g = model_zoo.GraphBuilder(seed)
    r = g.rng
    x = g.placeholder("input", [batch, 24, 24, 6])
    y = g.conv(x, (r.standard_normal((11, 11, 6, 8)) / 27).astype(np.float32),
               r.standard_normal(8).astype(np.float32), 1, "relu")
    y = g.conv(y, (r.standard_normal((3, 3, 8, 64)) / 8).astype(np.float32),
               r.standard_normal(64).astype(np.float32), 1, None, name="out")
    return g.artifacts(["input"], [y])


def test_stale_graph_is_refused_and_captured_again(cuda_engine):
    """A captured step carries the addresses of the scratch buffer and of the packed weight
    copies.  When an eager call makes the scratch buffer grow, or a weight is rewritten, the
    library refuses the old graph; GraphModel runs that step eagerly and captures again."""
    from tfjs_b200 import ops as tf
    be = cuda_engine.backend
    model_json, weights = _im2col_model(2)
    fast = GraphModel(model_json, weights, cuda_engine, replay=True)
    eager = GraphModel(model_json, weights, cuda_engine, replay=False)

    def step(seed):
        x = np.random.default_rng(seed).standard_normal((2, 24, 24, 6)).astype(np.float32)
        t = cuda_engine.make_tensor(x)
        got, want = fast.execute(t, ["out"])[0], eager.execute(t, ["out"])[0]
        a, b = got.dataSync(), want.dataSync()
        for v in (t, got, want):
            v.dispose()
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32)), seed
        return list(fast._replays.values())[0]

    assert [step(s)["state"] for s in range(3)] == ["warm", "ready", "ready"]
    graph = list(fast._replays.values())[0]["graph"]
    # a larger convolution of the same kind, eagerly: the scratch buffer is re-allocated
    r = np.random.default_rng(9)
    big = tf.tensor(r.standard_normal((16, 40, 40, 6)).astype(np.float32))
    f = tf.tensor((r.standard_normal((11, 11, 6, 8)) / 27).astype(np.float32))
    y = tf.conv2d(big, f, [1, 1], "same")
    y.dataSync()
    for t in (big, f, y):
        t.dispose()
    assert be.lib.tfjs_cuda_graph_launch(be.ctx, graph) == 5        # TFJS_CUDA_UNSUPPORTED
    assert b"stale" in be.lib.tfjs_cuda_last_error(be.ctx)
    st = step(3)
    assert st["state"] == "warm" and st["recaptures"] == 1
    assert [step(s)["state"] for s in (4, 5)] == ["ready", "ready"]
    # rewriting a weight drops its packed copy: stale again, and the new values are used
    name = [n for n, t in fast.weights.items() if t.shape == [3, 3, 8, 64]][0]
    new = np.random.default_rng(10).standard_normal((3, 3, 8, 64)).astype(np.float32)
    for gm in (fast, eager):
        dev = be.device_id(gm.weights[name].dataId)
        be.check(be.lib.tfjs_cuda_write(be.ctx, dev, new.ctypes.data_as(ctypes.c_void_p),
                                        new.nbytes))
    st = step(6)
    assert st["state"] == "warm" and st["recaptures"] == 2
    assert step(7)["state"] == "ready"
    fast.dispose()
    eager.dispose()
