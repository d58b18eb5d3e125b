"""The stem of MobileNetV2 (3-channel image, 3 x 3 stride-2 filter, 32 output channels) runs
as a direct fp32 kernel (`stem_conv3x3s2_kernel`) in the default math mode.

Against the CPU oracle (FusedConv2D.ts:26-95): the kernel performs the reference's fp32
multiply-adds in the reference's order (filter row, filter column, input channel; bias and
activation afterwards), so the bound is that of the last bit of each accumulation, far
inside the 2e-3 * max|ref| that bounds the TF32 product it replaces."""
import numpy as np
import pytest

from oracle import oracle as orc

pytestmark = pytest.mark.gpu


def _run(tf, backend, x, w, bias, pad, activation):
    ts = [tf.tensor(x), tf.tensor(w)] + ([tf.tensor(bias)] if bias is not None else [])
    backend.launch_log(True)
    backend.launch_log_take()
    y = tf.fused_conv2d(ts[0], ts[1], 2, pad, "NHWC", [1, 1], None,
                        ts[2] if bias is not None else None, activation)
    got = y.dataSync().reshape(y.shape)
    log = backend.launch_log_take()
    backend.launch_log(False)
    for t in ts + [y]:
        t.dispose()
    return got, log


@pytest.mark.parametrize("batch,h,w,pad,activation,with_bias", [
    (2, 224, 224, "same", "relu6", True),    # the layer itself (pad: bottom and right only)
    (3, 30, 36, "same", "relu", True),       # 15 output rows (a partial unit), 18 columns (a partial group)
    (1, 31, 32, "same", "linear", False),    # odd height: one padding row on top as well
    (5, 33, 40, "valid", "relu6", True),     # no padding; more units than fit one round on few rows
    (1, 8, 8, "same", "linear", True),       # a single unit
])
def test_stem_kernel_matches_the_oracle(cuda_engine, batch, h, w, pad, activation, with_bias):
    from tfjs_b200 import ops as tf
    r = np.random.default_rng(h * 1000 + w)
    x = r.standard_normal((batch, h, w, 3)).astype(np.float32)
    f = (r.standard_normal((3, 3, 3, 32)) / 5).astype(np.float32)
    bias = r.standard_normal(32).astype(np.float32) if with_bias else None
    backend = cuda_engine.backend
    before = backend.numDataIds()
    got, log = _run(tf, backend, x, f, bias, pad, activation)
    assert "stem_conv3x3s2_kernel" in log and "gemm" not in log, log
    assert backend.numDataIds() == before
    ref = orc.fused_conv2d(x, f, 2, pad, bias=bias, activation=activation)
    assert got.shape == ref.shape
    assert np.max(np.abs(got - ref)) <= 2e-6 * np.max(np.abs(ref))


def test_stem_kernel_keeps_nan_and_clamps(cuda_engine):
    from tfjs_b200 import ops as tf
    r = np.random.default_rng(1)
    x = (r.standard_normal((1, 16, 16, 3)) * 8).astype(np.float32)
    x[0, 4, 6, 1] = np.nan
    f = r.standard_normal((3, 3, 3, 32)).astype(np.float32)
    got, log = _run(tf, cuda_engine.backend, x, f, None, "same", "relu6")
    assert "stem_conv3x3s2_kernel" in log
    ref = orc.fused_conv2d(x, f, 2, "same", activation="relu6")
    assert np.array_equal(np.isnan(got), np.isnan(ref)) and np.isnan(got).any()
    ok = ~np.isnan(ref)
    assert got[ok].min() >= 0.0 and got[ok].max() <= 6.0
    assert np.max(np.abs(got[ok] - ref[ok])) <= 2e-5


def test_stem_kernel_with_a_folded_shortcut(cuda_engine):
    """conv + bias, Add of a shortcut, Relu as one launch of the same kernel."""
    from tfjs_b200 import ops as tf
    r = np.random.default_rng(4)
    x = r.standard_normal((2, 32, 32, 3)).astype(np.float32)
    f = (r.standard_normal((3, 3, 3, 32)) / 5).astype(np.float32)
    b = r.standard_normal(32).astype(np.float32)
    sc = r.standard_normal((2, 16, 16, 32)).astype(np.float32)
    backend = cuda_engine.backend
    ts = [tf.tensor(v) for v in (x, f, b, sc)]
    backend.launch_log(True)
    backend.launch_log_take()
    y = tf.fused_conv2d(ts[0], ts[1], 2, "same", "NHWC", [1, 1], None, ts[2], "linear")
    s = tf.add(y, ts[3])
    o = tf.relu(s)
    got = o.dataSync().reshape(o.shape)
    log = backend.launch_log_take()
    backend.launch_log(False)
    for t in ts + [y, s, o]:
        t.dispose()
    assert log.count("stem_conv3x3s2_kernel") == 1 and "add" not in log.lower(), log
    ref = orc.fused_conv2d(x, f, 2, "same", bias=b)
    ref = np.maximum(ref + sc, 0).astype(np.float32)
    assert np.max(np.abs(got - ref)) <= 2e-6 * np.max(np.abs(ref))


def test_shapes_the_stem_kernel_declines_take_the_tensor_core_path(cuda_engine):
    """An image width that is not a multiple of four (the bulk copies need 16-byte rows), a
    left padding column, 64 output channels or stride 1: the staged-row GEMM as before."""
    from tfjs_b200 import ops as tf
    r = np.random.default_rng(2)
    for (h, w, cout, stride_ok) in ((30, 30, 32, True), (31, 31, 32, True), (32, 32, 64, True)):
        x = r.standard_normal((2, h, w, 3)).astype(np.float32)
        f = (r.standard_normal((3, 3, 3, cout)) / 5).astype(np.float32)
        got, log = _run(tf, cuda_engine.backend, x, f, None, "same", "relu")
        assert "stem_conv3x3s2_kernel" not in log and "gemm_tf32" in log, log
        ref = orc.fused_conv2d(x, f, 2, "same", activation="relu")
        assert np.max(np.abs(got - ref)) <= 2e-3 * np.max(np.abs(ref))
