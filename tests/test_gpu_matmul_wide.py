"""Products whose 256 x 256 tiles would need between one and one and a half waves of CTA
pairs run on 256 x 384 tiles instead (`gemm_tf32_pair_kernel<..., BN=384>`: two N = 192
MMAs per K slice, one accumulator stage).  Results against the CPU oracle
(_FusedMatMul.ts:26-62) within the floating-point bound for TF32 inputs, 2e-3 * max|ref|."""
import numpy as np
import pytest

from oracle import oracle as orc

pytestmark = pytest.mark.gpu

TF32_TOL = 2e-3


def _sm_count():
    import torch
    return torch.cuda.get_device_properties(0).multi_processor_count


def _product(tf, backend, a, w, b, activation, heads=None):
    ts = [tf.tensor(v) for v in (a, w, b)]
    backend.launch_log(True)
    backend.launch_log_take()
    if heads is None:
        y = tf.fused_mat_mul(ts[0], ts[1], False, False, ts[2], activation)
    else:
        y = tf.mat_mul_heads(ts[0], ts[1], "split", heads, False, False, ts[2], activation)
    got = y.dataSync().reshape(y.shape)
    log = backend.launch_log_take()
    backend.launch_log(False)
    for t in ts + [y]:
        t.dispose()
    return got, log


@pytest.mark.parametrize("m,k,n,activation", [
    (4864, 256, 1152, "linear"),     # whole tiles: 19 x 3 of 256 x 384
    (4800, 260, 1000, "relu"),       # ragged in every dimension (K tail, partial last tiles)
    (8192, 768, 768, "relu6"),       # the attention output projection of BERT-base, batch 64
])
def test_wide_tiles_match_the_oracle(cuda_engine, m, k, n, activation):
    from tfjs_b200 import ops as tf
    if _sm_count() != 148:
        pytest.skip("tile counts chosen for 148 SMs")
    r = np.random.default_rng(m + n)
    a = r.standard_normal((m, k)).astype(np.float32)
    w = (r.standard_normal((k, n)) / np.sqrt(k)).astype(np.float32)
    b = (r.standard_normal(n) * 0.1).astype(np.float32)
    got, log = _product(tf, cuda_engine.backend, a, w, b, activation)
    assert "BN=384" in log, log
    ref = orc.fused_matmul(a, w, False, False, bias=b, activation=activation)
    assert np.max(np.abs(got - ref)) <= TF32_TOL * np.max(np.abs(ref))
    # every tile was written: no element left at the pool's previous contents
    assert np.all(np.isfinite(got))


def test_wide_tiles_with_heads_split_store(cuda_engine):
    from tfjs_b200 import ops as tf
    if _sm_count() != 148:
        pytest.skip("tile counts chosen for 148 SMs")
    B, S, H, D = 64, 128, 12, 64
    r = np.random.default_rng(5)
    a = r.standard_normal((B * S, 256)).astype(np.float32)
    w = (r.standard_normal((256, H * D)) / 16).astype(np.float32)
    b = (r.standard_normal(H * D) * 0.1).astype(np.float32)
    got, log = _product(tf, cuda_engine.backend, a, w, b, "linear", [B, S, H, D])
    assert "BN=384" in log, log
    ref = orc.fused_matmul(a, w, False, False, bias=b).reshape(B, S, H, D).transpose(0, 2, 1, 3)
    assert got.shape == (B, H, S, D)
    assert np.max(np.abs(got - ref)) <= TF32_TOL * np.max(np.abs(ref))
