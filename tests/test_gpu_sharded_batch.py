"""The batch split over replicas (B200 only): two ranks, each with its own backend
context, take contiguous halves of a batch, execute, and rank 0 concatenates the halves
read back from both; the result must be the bits of one replica running the whole batch.

The ranks run as two processes.  With two or more GPUs each rank takes its own GPU; on a
one-GPU box both contexts share device 0 (the kernels of the two ranks do not wait on one
another, so sharing a device only serialises them).  The rendezvous is gloo on 127.0.0.1;
nothing crosses NVLink.
"""
import json
import os
import subprocess
import sys
import textwrap

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

RANK_SCRIPT = """
    import json, os, sys
    import numpy as np
    rank = int(os.environ["RANK"])
    import ctypes
    from tfjs_b200 import _cabi
    n = ctypes.c_int()
    _cabi.load().tfjs_cuda_device_count(ctypes.byref(n))
    os.environ["TFJS_CUDA_DEVICE_ORDINAL"] = str(rank % max(n.value, 1))
    import tfjs_b200
    from tfjs_b200 import model_zoo
    from tfjs_b200.replicas import ReplicaGroup, sharded_execute
    eng = tfjs_b200.ENGINE
    eng.set_backend("cuda")
    kind, batch, out_path = sys.argv[1], int(sys.argv[2]), sys.argv[3]
    r = np.random.default_rng(77)
    if kind == "mobilenet":
        build = lambda b: model_zoo.mobilenet_v2(b, size=96)
        feeds = {"input": r.uniform(-1, 1, (batch, 96, 96, 3)).astype(np.float32)}
        out = "logits"
    else:
        build = lambda b: model_zoo.bert_encoder(b, seq=64, layers=2)
        feeds = {"input_ids": r.integers(0, 30522, (batch, 64)).astype(np.int32),
                 "attention_mask": np.ones((batch, 64), np.float32)}
        out = "sequence_output"
    g = ReplicaGroup()
    got = sharded_execute(eng, build, feeds, out, g)
    if g.rank == 0:
        np.save(out_path, got)
        print("RESULT " + json.dumps({"world": g.world, "shape": list(got.shape),
                                      "devices": n.value}))
    else:
        assert got is None
    g.close()
"""


@pytest.mark.parametrize("kind,batch", [("mobilenet", 7), ("bert", 4)])
def test_two_replicas_reproduce_the_one_gpu_result(cuda_engine, tmp_path, kind, batch):
    from tfjs_b200 import model_zoo
    from tfjs_b200.replicas import ReplicaGroup, sharded_execute
    script = tmp_path / "rank.py"
    script.write_text(textwrap.dedent(RANK_SCRIPT))
    out_path = str(tmp_path / "gathered.npy")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", "29541", str(script), kind, str(batch),
           out_path]
    res = subprocess.run(cmd, cwd=ROOT, env=dict(os.environ, PYTHONPATH=ROOT),
                         capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-3000:]
    line = [l for l in res.stdout.splitlines() if l.startswith("RESULT ")]
    assert len(line) == 1, res.stdout[-2000:]
    info = json.loads(line[0][7:])
    assert info["world"] == 2
    gathered = np.load(out_path)
    # the whole batch on one replica, in this process
    r = np.random.default_rng(77)
    if kind == "mobilenet":
        build = lambda b: model_zoo.mobilenet_v2(b, size=96)
        feeds = {"input": r.uniform(-1, 1, (batch, 96, 96, 3)).astype(np.float32)}
        out = "logits"
    else:
        build = lambda b: model_zoo.bert_encoder(b, seq=64, layers=2)
        feeds = {"input_ids": r.integers(0, 30522, (batch, 64)).astype(np.int32),
                 "attention_mask": np.ones((batch, 64), np.float32)}
        out = "sequence_output"
    whole = sharded_execute(cuda_engine, build, feeds, out, ReplicaGroup(0, 1))
    assert gathered.shape == whole.shape and gathered.shape[0] == batch
    # units are independent and a kernel's result for a unit does not depend on the batch it
    # is part of, except where the batch size changes the GEMM's tile schedule (another
    # summation order under the K-split tail): bound by TF32 noise, not bit identity
    denom = float(np.max(np.abs(whole)))
    assert float(np.max(np.abs(gathered - whole))) / denom <= 2e-3
