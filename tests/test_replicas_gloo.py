"""The multi-GPU host logic (one process per GPU, batch-sharded replicas) run as two
gloo ranks on CPU: batch split, barrier, max over ranks, host-side gather, and the
benchmark's reference arm under a two-rank launch."""
import json
import os
import subprocess
import sys
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _launch(script_args, port):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", str(port)] + script_args
    env = dict(os.environ, PYTHONPATH=ROOT, OMP_NUM_THREADS="2")
    return subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)


def test_shard_range_covers_batch_once():
    from tfjs_b200.replicas import shard_range
    for total in (0, 1, 7, 128, 256):
        for world in (1, 2, 3, 8):
            seen = []
            for r in range(world):
                lo, hi = shard_range(total, world, r)
                assert 0 <= lo <= hi <= total
                seen += list(range(lo, hi))
            assert seen == list(range(total))


def test_two_rank_group(tmp_path):
    script = tmp_path / "ranks.py"
    script.write_text(textwrap.dedent("""
        import json, sys
        import numpy as np
        from tfjs_b200.replicas import ReplicaGroup, shard_range
        g = ReplicaGroup()
        lo, hi = shard_range(10, g.world, g.rank)
        local = np.arange(lo, hi, dtype=np.float32).reshape(-1, 1) * 2.0   # "logits" of my slice
        g.barrier()
        slowest = g.max_over_ranks(1.5 if g.rank == 1 else 0.5)
        total = g.sum_over_ranks(hi - lo)
        out = g.gather_to_root(local)
        if g.rank == 0:
            print("RESULT " + json.dumps({"world": g.world, "slowest": slowest, "total": total,
                                          "gathered": out.reshape(-1).tolist()}))
        else:
            assert out is None
        g.close()
    """))
    res = _launch([str(script)], 29533)
    assert res.returncode == 0, res.stderr[-2000:]
    line = [l for l in res.stdout.splitlines() if l.startswith("RESULT ")]
    assert len(line) == 1
    got = json.loads(line[0][7:])
    assert got == {"world": 2, "slowest": 1.5, "total": 10.0,
                   "gathered": [float(2 * i) for i in range(10)]}


def test_bench_reference_arm_two_ranks():
    """Under a 2-rank launch rank 0 alone prints the reference line."""
    res = _launch(["bench.py", "--impl", "reference", "--gpus", "2", "--steps", "1", "--warmup", "0",
                   "--cpu-sample", "1"], 29534)
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [l for l in res.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["n_gpus"] == 2 and d["value"] > 0
    assert d["cpu_baseline"]["kind"] == "port" and d["e2e"]["h2d_bytes_per_step"] == 0
