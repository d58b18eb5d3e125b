"""The configurations bench.py times, at their full sizes, against the CPU oracle (B200 only).

The library picks kernel instantiations from the problem size (tile width, swapped
operands, K-split tail, sixteen-warp epilogue ...), so a model checked at batch 2 has not
checked the kernels that run at batch 256.  Images / sequences of a batch are independent,
which keeps the scalar oracle affordable: it runs a handful of units.

(a) end to end, exactly as bench.py runs a step: GraphModel(replay=True) on the seeded
    bench batch, three executes (eager, capture, replay); units 0, 1 and the last of the
    replayed result are compared with the oracle's result for those units: bound
    1e-2 * max|ref| (TF32 rounding noise is a random walk over ~50 layers) and, for the
    classifiers, identical top-1.
(b) per layer at the full batch: the oracle runs three units; every compute node is then
    run on the GPU at the bench batch with the ORACLE's inputs for that node, tiled to the
    full batch, so only that kernel's own error shows, and every unit of its output is
    compared on the device with the oracle's output for the unit it repeats: bound
    2e-3 * max|ref| (TF32 operands, fp32 accumulation).
"""
import numpy as np
import pytest

import bench
from oracle import graph_oracle
from tfjs_b200 import graph_model, ops
from tfjs_b200.graph_model import GraphModel

pytestmark = pytest.mark.gpu
TOL = 2e-3          # per layer, oracle inputs
DRIFT_TOL = 1e-2    # end to end

CONFIGS = [("mobilenet_v2", 256), ("mobilenet_v2", 64), ("mobilenet_v2", 1), ("resnet50", 128),
           ("bert", 64)]


def _dtype(v):
    return "int32" if v.dtype == np.int32 else "float32"


def _same_float_weights(model_a, bytes_a, model_b, bytes_b):
    """The generators are seeded: models built for two batch sizes must hold the same
    trained tensors (only shape constants differ)."""
    wa = graph_oracle.decode_weights(bytes_a, model_a["weightsManifest"][0]["weights"])
    wb = graph_oracle.decode_weights(bytes_b, model_b["weightsManifest"][0]["weights"])
    assert list(wa) == list(wb)
    for name in wa:
        if wa[name].dtype == np.float32:
            assert np.array_equal(wa[name], wb[name]), name


def _oracle_units(kind, batch, feeds, units):
    """Oracle outputs of every node for the given units of the bench batch."""
    small_json, small_weights = bench.build_model(kind, len(units))
    small_feeds = {k: np.ascontiguousarray(v[units]) for k, v in feeds.items()}
    return small_json, small_weights, graph_oracle.run(small_json, small_weights, small_feeds)


@pytest.mark.parametrize("kind,batch", CONFIGS, ids=["%s_b%d" % c for c in CONFIGS])
def test_replayed_bench_step_matches_oracle_on_sampled_units(cuda_engine, kind, batch):
    eng = cuda_engine
    out_name = bench.WORKLOADS[kind]["out"]
    model_json, weights = bench.build_model(kind, batch)
    feeds = bench.make_feeds(kind, batch, 1000)
    units = sorted(set([0, min(1, batch - 1), batch - 1]))
    small_json, small_weights, ref = _oracle_units(kind, batch, feeds, units)
    _same_float_weights(model_json, weights, small_json, small_weights)

    gm = GraphModel(model_json, weights, eng, replay=True)
    ins = {k: eng.make_tensor(v, list(v.shape), _dtype(v)) for k, v in feeds.items()}
    # eager, capture (repeated with a larger arena if the first one fragments), then replays
    for _ in range(5):
        gm.execute(ins, [out_name])[0].dispose()
        state = list(gm._replays.values())[0]
        if state["state"] != "warm":
            break
    assert state["state"] == "ready", state.get("why")
    launches = eng.backend.launch_count()
    y = gm.execute(ins, [out_name])[0]              # a replay
    got = y.arraySync()
    y.dispose()
    assert eng.backend.launch_count() > launches
    for t in ins.values():
        t.dispose()
    gm.dispose()

    want = ref[out_name]
    got_units = got[units]
    assert got_units.shape == want.shape
    denom = float(np.max(np.abs(want)))
    err = float(np.max(np.abs(got_units.astype(np.float64) - want))) / denom
    assert err <= DRIFT_TOL, (kind, batch, err)
    if kind != "bert":
        assert np.array_equal(got_units.argmax(-1), want.argmax(-1))


def _tile_units(t, n_units, batch):
    """Device tensor whose leading axis holds `batch` units, unit i repeating unit
    i % n_units of `t` (leading axis = n_units * rows per unit)."""
    rows = t.shape[0] // n_units
    reps = -(-batch // n_units)
    tiled = ops.tile(t, [reps] + [1] * (len(t.shape) - 1))
    if reps * n_units == batch:
        return tiled
    out = ops.slice(tiled, [0] * len(t.shape), [rows * batch] + list(t.shape[1:]))
    tiled.dispose()
    return out


@pytest.mark.parametrize("kind,batch", [c for c in CONFIGS if c[1] > 1],
                         ids=["%s_b%d" % c for c in CONFIGS if c[1] > 1])
def test_every_layer_at_the_bench_batch_matches_oracle(cuda_engine, kind, batch):
    eng = cuda_engine
    model_json, weights = bench.build_model(kind, batch)
    feeds = bench.make_feeds(kind, batch, 1000)
    n_units = 3
    small_json, small_weights, ref = _oracle_units(kind, batch, feeds, list(range(n_units)))
    gm = GraphModel(model_json, weights, eng, replay=False)
    worst = ("", 0.0)
    checked = 0
    for d in model_json["modelTopology"]["node"]:
        if d["op"] in ("Const", "Placeholder"):
            continue
        node = graph_model.Node(d)
        made, ins = [], []
        for i in node.inputs:
            src = i.split(":")[0]
            if src in gm.weights:
                ins.append(gm.weights[src])
                continue
            v = ref[src]
            assert v.shape[0] % n_units == 0, (src, v.shape)
            small = eng.make_tensor(v, list(v.shape), _dtype(v))
            big = _tile_units(small, n_units, batch)
            made += [small, big]
            ins.append(big)
        out = graph_model.execute_op(node, ins)
        r = ref[node.name]
        assert r.shape[0] % n_units == 0 and out.shape[0] * n_units == r.shape[0] * batch, \
            (node.name, out.shape, r.shape)
        want_small = eng.make_tensor(r, list(r.shape), _dtype(r))
        want = _tile_units(want_small, n_units, batch)
        if out.dtype == "float32":
            diff = ops.sub(out, want)
            mag = ops.abs(diff)
            top = ops.max(mag)
            err = float(top.dataSync()[0]) / (float(np.max(np.abs(r))) or 1.0)
            made += [diff, mag, top]
        else:
            err = 0.0 if np.array_equal(out.arraySync(), want.arraySync()) else 1.0
        made += [out, want_small, want]
        for t in made:
            t.dispose()
        checked += 1
        if not err <= worst[1]:          # also catches NaN
            worst = (node.name + ":" + node.op, err)
    gm.dispose()
    assert checked > 50
    assert worst[1] <= TOL, worst
