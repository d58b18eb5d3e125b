"""One attention layer as one launch (`tfjs_cuda_fused_attention`, kernel `_FusedAttention`):
softmax(q k^T * scale + mask) v for heads of 128 positions x 64 features, stored with the
heads merged.

Checked against the CPU oracle's chain of the reference's kernels (BatchMatMul.ts:29-113,
Multiply.ts, Add.ts, Softmax.ts:50-67, Transpose) within the floating-point bound for TF32
products, 2e-3 * max|ref|, and against the separate launches of this library, from which it
may differ only by the order of the softmax's fp32 sum."""
import numpy as np
import pytest

from oracle import oracle as orc

pytestmark = pytest.mark.gpu

TF32_TOL = 2e-3
# against the separate launches: a probability that differs in its last fp32 bit (the sum's
# order) can round to the neighbouring TF32 value, 2^-11 of it
SEP_TOL = 1e-3
S, D = 128, 64


def _oracle(q, k, v, scale, mask):
    s = orc.batch_matmul(q, k, False, True)
    if scale is not None:
        s = orc.binary("mul", s, np.float32(scale))
    if mask is not None:
        s = orc.binary("add", s, mask)
    p = orc.softmax(s)
    o = orc.batch_matmul(p, v)
    return np.ascontiguousarray(o.transpose(0, 2, 1, 3))


def _inputs(seed, B, H, spread=1.0):
    r = np.random.default_rng(seed)
    q = (r.standard_normal((B, H, S, D)) * spread).astype(np.float32)
    k = r.standard_normal((B, H, S, D)).astype(np.float32)
    v = r.standard_normal((B, H, S, D)).astype(np.float32)
    return q, k, v


def _fused(tf, backend, q, k, v, scale, mask):
    ts = [tf.tensor(a) for a in (q, k, v)] + ([tf.tensor(mask)] if mask is not None else [])
    backend.launch_log(True)
    backend.launch_log_take()
    y = tf.fused_attention(ts[0], ts[1], ts[2], scale, ts[3] if mask is not None else None)
    got = y.dataSync().reshape(y.shape)
    log = backend.launch_log_take()
    backend.launch_log(False)
    for t in ts + [y]:
        t.dispose()
    return got, log


def _separate(tf, q, k, v, scale, mask):
    B, H = q.shape[:2]
    ts = [tf.tensor(a) for a in (q, k, v)] + ([tf.tensor(mask)] if mask is not None else [])
    s = tf.mat_mul(ts[0], ts[1], False, True)
    p = tf.softmax_scaled_masked(s, scale, ts[3] if mask is not None else None)
    o = tf.mat_mul_heads(p, ts[2], "merge", [B, S, H, D])
    sep = o.dataSync().reshape(B, S, H, D)
    for t in ts + [s, p, o]:
        t.dispose()
    return sep


@pytest.mark.parametrize("B,H,scale,masked", [
    (2, 12, 0.125, True),     # fewer heads than SMs
    (1, 1, None, False),      # a single unit, no scale, no mask
    (16, 12, 0.125, True),    # 192 units: some CTAs take two, which exercises both slots
    (40, 12, 0.125, False),   # 480 units: up to four per CTA, slots reused
])
def test_fused_attention_matches_the_oracle(cuda_engine, B, H, scale, masked):
    from tfjs_b200 import ops as tf
    # scores of order one either way (TF32 rounding of larger scores moves the probabilities
    # by more than the bound, in the separate launches as well)
    q, k, v = _inputs(B * 100 + H, B, H, spread=1.0 if scale is not None else 0.125)
    mask = None
    if masked:
        r = np.random.default_rng(7)
        mask = np.where(r.random((B, 1, 1, S)) < 0.2, -10000.0, 0.0).astype(np.float32)
    backend = cuda_engine.backend
    before = backend.numDataIds()
    got, log = _fused(tf, backend, q, k, v, scale, mask)
    assert log.count("attention_kernel") == 1 and "gemm" not in log and "softmax" not in log, log
    assert backend.numDataIds() == before
    ref = _oracle(q, k, v, scale, mask)
    assert got.shape == (B, S, H, D)
    assert np.max(np.abs(got - ref)) <= TF32_TOL * np.max(np.abs(ref))


def test_fused_attention_against_the_separate_launches(cuda_engine):
    """Same products and roundings as batchMatMul + softmax_scaled_masked + the heads-merging
    product; only the softmax's sum is formed in another order (most results are equal
    bit for bit)."""
    from tfjs_b200 import ops as tf
    B, H = 4, 12
    q, k, v = _inputs(3, B, H, spread=2.0)
    mask = np.zeros((B, 1, 1, S), np.float32)
    mask[:, :, :, 100:] = -10000.0
    got, _ = _fused(tf, cuda_engine.backend, q, k, v, 0.125, mask)
    sep = _separate(tf, q, k, v, 0.125, mask)
    assert np.mean(got != sep) < 0.25
    assert np.max(np.abs(got - sep)) <= SEP_TOL * np.max(np.abs(sep))
    # masked keys carry no weight: the result equals attention over the first 100 keys
    ref = _oracle(q[:, :, :, :], k[:, :, :100], v[:, :, :100], 0.125, None)
    assert np.max(np.abs(got - ref)) <= TF32_TOL * np.max(np.abs(ref))


def test_fused_attention_nan_and_large_scores(cuda_engine):
    """A NaN in q poisons exactly its row; scores of several hundred neither overflow nor
    lose the row's largest term."""
    from tfjs_b200 import ops as tf
    B, H = 1, 2
    q, k, v = _inputs(11, B, H, spread=6.0)
    q[0, 1, 5, 3] = np.nan
    got, _ = _fused(tf, cuda_engine.backend, q, k, v, None, None)
    assert np.all(np.isnan(got[0, 5, 1, :]))
    ok = np.ones((B, S, H), bool)
    ok[0, 5, 1] = False
    assert np.all(np.isfinite(got[ok]))
    # (TF32 rounding of scores this large moves the probabilities by percents against an
    # fp32 evaluation, in the separate launches as well: those are the yardstick here)
    sep = _separate(tf, q, k, v, None, None)
    assert np.all(np.isnan(sep[0, 5, 1, :]))
    assert np.max(np.abs(got[ok] - sep[ok])) <= SEP_TOL * np.max(np.abs(sep[ok]))


def test_other_shapes_are_declined_and_nothing_is_launched(cuda_engine):
    from tfjs_b200 import ops as tf, _cabi
    backend = cuda_engine.backend
    r = np.random.default_rng(2)
    for shape in ((2, 4, 64, 64), (2, 4, 128, 32)):
        ts = [tf.tensor(r.standard_normal(shape).astype(np.float32)) for _ in range(3)]
        before = backend.numDataIds()
        backend.launch_log(True)
        backend.launch_log_take()
        with pytest.raises(_cabi.CudaError) as e:
            tf.fused_attention(ts[0], ts[1], ts[2], 0.125, None)
        assert e.value.code == _cabi.UNSUPPORTED
        assert backend.launch_log_take().strip() == ""
        backend.launch_log(False)
        assert backend.numDataIds() == before
        for t in ts:
            t.dispose()
    # a mask with one row per query is not one row per head
    ts = [tf.tensor(r.standard_normal((1, 2, S, D)).astype(np.float32)) for _ in range(3)]
    m = tf.tensor(np.zeros((1, 2, S, S), np.float32))
    with pytest.raises(_cabi.CudaError):
        tf.fused_attention(ts[0], ts[1], ts[2], 0.125, m)
    for t in ts + [m]:
        t.dispose()
