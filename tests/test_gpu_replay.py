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
