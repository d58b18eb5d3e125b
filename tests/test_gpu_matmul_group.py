"""Products that share their `a` operand (the query, key and value projections of an
attention layer) launched as one group: `tfjs_cuda_fused_matmul_group`, reached through the
backend's pending launches (`PendingMatMul`).

Each member's result must be the one its own launch gives (bit for bit: the same K steps
in the same order feed the same fp32 accumulators) and agree with the CPU oracle
(_FusedMatMul.ts:26-62) within the floating-point bound for TF32 inputs, 2e-3 * max|ref|.
"""
from ctypes import byref, c_int32, c_void_p

import numpy as np
import pytest

from oracle import oracle as orc

pytestmark = pytest.mark.gpu

TF32_TOL = 2e-3


def _weights(r, k, n, count):
    return [((r.standard_normal((k, n)) / np.sqrt(k)).astype(np.float32),
             (r.standard_normal(n) * 0.1).astype(np.float32)) for _ in range(count)]


def _run(tf, backend, a, ws, activation, heads, grouped, use_bias=True):
    backend.group_matmuls = grouped
    made = []
    try:
        a0, zero = tf.tensor(a), tf.tensor(np.float32(0))
        at = tf.add(a0, zero)                          # an activation, not a weight
        made += [a0, zero, at]
        outs = []
        for w, b in ws:
            wt, bt = tf.tensor(w), (tf.tensor(b) if use_bias else None)
            made += [t for t in (wt, bt) if t is not None]
            if heads is None:
                outs.append(tf.fused_mat_mul(at, wt, False, False, bt, activation))
            else:
                outs.append(tf.mat_mul_heads(at, wt, "split", heads, False, False, bt, activation))
        backend.launch_log(True)
        backend.launch_log_take()
        vals = [o.dataSync().reshape(o.shape) for o in outs]
        log = backend.launch_log_take()
        backend.launch_log(False)
        for o in outs:
            o.dispose()
        return vals, log
    finally:
        backend.group_matmuls = True
        for t in made:
            t.dispose()


@pytest.mark.parametrize("m,k,n,count,activation", [
    (1024, 256, 768, 3, "linear"),      # the attention projections' shape, scaled down
    (640, 320, 384, 2, "relu"),         # ragged tile counts: M and N not multiples of 256
    (300, 128, 1000, 4, "relu6"),       # four members, N with a partial last tile
])
def test_group_matches_separate_launches_and_oracle(cuda_engine, m, k, n, count, activation):
    from tfjs_b200 import ops as tf
    r = np.random.default_rng(m + n)
    a = r.standard_normal((m, k)).astype(np.float32)
    ws = _weights(r, k, n, count)
    backend = cuda_engine.backend
    before = backend.numDataIds()
    got, log = _run(tf, backend, a, ws, activation, None, True)
    assert log.count("gemm_tf32_pair_kernel<A_MODE=0,EW=8,GROUP=1>") == 1, log
    assert "gemm_tf32_kernel<" not in log
    sep, sep_log = _run(tf, backend, a, ws, activation, None, False)
    assert "GROUP=1" not in sep_log
    assert backend.numDataIds() == before
    for g, s, (w, b) in zip(got, sep, ws):
        assert np.array_equal(g.view(np.uint32), s.view(np.uint32)), float(np.max(np.abs(g - s)))
        ref = orc.fused_matmul(a, w, False, False, bias=b, activation=activation)
        assert np.max(np.abs(g - ref)) <= TF32_TOL * np.max(np.abs(ref))


def test_group_with_heads_split_store(cuda_engine):
    from tfjs_b200 import ops as tf
    B, S, H, D = 4, 128, 6, 64
    r = np.random.default_rng(3)
    a = r.standard_normal((B * S, 192)).astype(np.float32)
    ws = _weights(r, 192, H * D, 3)
    backend = cuda_engine.backend
    got, log = _run(tf, backend, a, ws, "linear", [B, S, H, D], True)
    assert log.count("GROUP=1") == 1, log
    sep, _ = _run(tf, backend, a, ws, "linear", [B, S, H, D], False)
    for g, s, (w, b) in zip(got, sep, ws):
        assert g.shape == (B, H, S, D)
        assert np.array_equal(g.view(np.uint32), s.view(np.uint32))
        ref = orc.fused_matmul(a, w, False, False, bias=b)
        ref = ref.reshape(B, S, H, D).transpose(0, 2, 1, 3)
        assert np.max(np.abs(g - ref)) <= TF32_TOL * np.max(np.abs(ref))


def test_only_like_products_group_and_a_dropped_member_is_skipped(cuda_engine):
    """Members must agree in every dimension; a product disposed before the group launches
    is left out; a lone product launches on its own."""
    from tfjs_b200 import ops as tf
    r = np.random.default_rng(9)
    a = r.standard_normal((512, 256)).astype(np.float32)
    (w1, b1), (w2, b2), (w3, b3) = _weights(r, 256, 512, 3)
    w4 = (r.standard_normal((256, 384)) / 16).astype(np.float32)
    b4 = (r.standard_normal(384) * 0.1).astype(np.float32)
    backend = cuda_engine.backend
    ts = [tf.tensor(v) for v in (a, w1, b1, w2, b2, w3, b3, w4, b4, np.float32(0))]
    at = tf.add(ts[0], ts[9])
    y1 = tf.fused_mat_mul(at, ts[1], False, False, ts[2], "linear")
    y2 = tf.fused_mat_mul(at, ts[3], False, False, ts[4], "linear")
    y3 = tf.fused_mat_mul(at, ts[5], False, False, ts[6], "linear")
    y4 = tf.fused_mat_mul(at, ts[7], False, False, ts[8], "linear")     # other width
    y3.dispose()                                                         # never needed
    backend.launch_log(True)
    backend.launch_log_take()
    v1 = y1.dataSync().reshape(y1.shape)
    log1 = backend.launch_log_take()
    v4 = y4.dataSync().reshape(y4.shape)
    log4 = backend.launch_log_take()
    v2 = y2.dataSync().reshape(y2.shape)        # already computed with y1
    log2 = backend.launch_log_take()
    backend.launch_log(False)
    assert log1.count("GROUP=1") == 1 and "GROUP=1" not in log4 and "gemm" not in log2, (log1, log4, log2)
    for v, w, b in ((v1, w1, b1), (v2, w2, b2), (v4, w4, b4)):
        ref = orc.fused_matmul(a, w, False, False, bias=b)
        assert np.max(np.abs(v - ref)) <= TF32_TOL * np.max(np.abs(ref))
    for t in ts + [at, y1, y2, y4]:
        t.dispose()


def test_c_abi_refuses_what_the_grouped_kernel_does_not_take(cuda_engine):
    """Straight through the C ABI: narrow outputs are reported as unsupported (the caller
    launches the members one by one), bad counts as invalid."""
    from tfjs_b200 import _cabi
    be = cuda_engine.backend
    lib = be.lib

    def upload(arr):
        out = c_int32()
        be.check(lib.tfjs_cuda_alloc(be.ctx, arr.nbytes, byref(out)))
        be.check(lib.tfjs_cuda_write(be.ctx, out.value, arr.ctypes.data_as(c_void_p), arr.nbytes))
        return out.value

    r = np.random.default_rng(1)
    m, k, n = 256, 64, 96
    a = upload(r.standard_normal((m, k)).astype(np.float32))
    bs = [upload(r.standard_normal((k, n)).astype(np.float32)) for _ in range(2)]
    outs = []
    for _ in range(2):
        o = c_int32()
        be.check(lib.tfjs_cuda_alloc(be.ctx, m * n * 4, byref(o)))
        outs.append(o.value)
    p = _cabi.MatMulParams()
    p.batch_a = p.batch_b = 1
    p.m, p.n, p.k = m, n, k
    arr = c_int32 * 2
    rc = lib.tfjs_cuda_fused_matmul_group(be.ctx, byref(p), a, 2, arr(*bs), None, 0, 0, 0, arr(*outs))
    assert rc == _cabi.UNSUPPORTED
    rc = lib.tfjs_cuda_fused_matmul_group(be.ctx, byref(p), a, 1, arr(*bs), None, 0, 0, 0, arr(*outs))
    assert rc not in (0, _cabi.UNSUPPORTED)
    for i in [a] + bs + outs:
        be.check(lib.tfjs_cuda_free(be.ctx, i))
