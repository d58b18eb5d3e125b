"""FusedDepthwiseConv2D followed by a 1x1 FusedConv2D (the tail of an inverted-residual
block) as one launch: `tfjs_cuda_fused_depthwise_project`, reached through the backend's
pending launches.

Every case is run three ways on the same seeded inputs: folded (one launch), as the two
separate kernels (TFJS_CUDA_NO_DW_PROJECT semantics, `fuse_depthwise_project = False`),
and through the CPU oracle (FusedDepthwiseConv2D.ts:25-61 then FusedConv2D.ts:26-95, Add,
Relu6).  Folded and separate must agree bit for bit: the folded kernel performs the same
fp32 operations per element and rounds the projection's operand to TF32 the way the TMA
unit does for the separate kernel.  Against the oracle the bound is the floating-point one,
2e-3 * max|ref| for TF32 tensor-core inputs.
"""
import zlib

import numpy as np
import pytest

from oracle import oracle as orc

pytestmark = pytest.mark.gpu

TF32_TOL = 2e-3

# name: (x shape, projection channels, depthwise activation, depthwise bias, projection bias,
#        shortcut, trailing activation[, depthwise stride])
CASES = {
    # MobileNetV2 block shapes (batch reduced): 112 / 56 / 28 / 14 / 7 maps
    "b1_112_32_16": ((2, 112, 112, 32), 16, "relu6", "vec", "vec", False, None),
    "b3_56_144_24_res": ((2, 56, 56, 144), 24, "relu6", "vec", "vec", True, None),
    "b5_28_192_32_res": ((3, 28, 28, 192), 32, "relu6", "vec", "vec", True, None),
    "b8_14_384_64_res": ((3, 14, 14, 384), 64, "relu6", "vec", "vec", True, None),
    "b11_14_384_96": ((2, 14, 14, 384), 96, "relu6", "vec", "vec", False, None),
    "b13_14_576_96_res": ((2, 14, 14, 576), 96, "relu6", "vec", "vec", True, None),
    "b16_7_960_160_res": ((5, 7, 7, 960), 160, "relu6", "vec", "vec", True, None),
    "b17_7_960_320": ((3, 7, 7, 960), 320, "relu6", "vec", "vec", False, None),
    # ragged sizes: maps that no tile divides, channel counts that are not multiples of 32,
    # a single image for the two-image tile, projections narrower than one MMA block
    "ragged_37x23_40_8": ((1, 37, 23, 40), 8, "relu", "vec", "vec", False, None),
    "ragged_19x19_100_44": ((3, 19, 19, 100), 44, "relu6", "vec", None, True, "relu"),
    "ragged_5x6_36_12": ((1, 5, 6, 36), 12, "linear", None, "vec", False, None),
    "one_image_7x7": ((1, 7, 7, 64), 264, "relu6", "scalar", "scalar", True, "relu6"),
    "wide_60x60_32_160": ((1, 60, 60, 32), 160, "relu6", "vec", "vec", False, "relu"),
    "linear_dw_no_bias": ((2, 16, 16, 64), 32, "linear", None, None, False, None),
    # the strided blocks of MobileNetV2: 112 -> 56, 56 -> 28, 28 -> 14, 14 -> 7
    "b2_s2_112_96_24": ((2, 112, 112, 96), 24, "relu6", "vec", "vec", False, None, 2),
    "b4_s2_56_144_32": ((2, 56, 56, 144), 32, "relu6", "vec", "vec", False, None, 2),
    "b7_s2_28_192_64": ((3, 28, 28, 192), 64, "relu6", "vec", "vec", False, None, 2),
    "b14_s2_14_576_160": ((3, 14, 14, 576), 160, "relu6", "vec", "vec", False, None, 2),
    "ragged_s2_37x23_40_8": ((1, 37, 23, 40), 8, "relu", "vec", "vec", True, "relu", 2),
    "ragged_s2_9x9_36_12": ((3, 9, 9, 36), 12, "linear", None, "vec", False, None, 2),
}


def _case(name):
    c = CASES[name]
    return c if len(c) == 8 else c + (1,)


def _inputs(name):
    xs, n, dw_act, dw_bias, pw_bias, with_add, post, stride = _case(name)
    r = np.random.default_rng(zlib.crc32(name.encode()) % 100000)
    c = xs[3]
    x = r.standard_normal(xs).astype(np.float32)
    wd = (r.standard_normal((3, 3, c, 1)) / 3).astype(np.float32)
    wp = (r.standard_normal((1, 1, c, n)) / np.sqrt(c)).astype(np.float32)

    def bias(kind, length):
        if kind is None:
            return None
        if kind == "scalar":
            return (r.standard_normal(1) * 0.1).astype(np.float32)
        return (r.standard_normal(length) * 0.1).astype(np.float32)

    bd, bp = bias(dw_bias, c), bias(pw_bias, n)
    out_hw = (-(-xs[1] // stride), -(-xs[2] // stride))
    shortcut = (r.standard_normal((xs[0],) + out_hw + (n,)).astype(np.float32)
                if with_add else None)
    return x, wd, bd, wp, bp, shortcut


def _block(tf, name, arrays):
    xs, n, dw_act, _, _, with_add, post, stride = _case(name)
    x, wd, bd, wp, bp, shortcut = arrays
    made = []

    def T(a):
        if a is None:
            return None
        t = tf.tensor(a)
        made.append(t)
        return t

    # x comes from a device kernel (an activation, not a weight)
    x0 = T(x)
    xt = tf.add(x0, T(np.float32(0)))
    made.append(xt)
    h = tf.fused_depthwise_conv2d(xt, T(wd), stride, "same", "NHWC", [1, 1], None, T(bd), dw_act)
    y = tf.fused_conv2d(h, T(wp), 1, "same", "NHWC", [1, 1], None, T(bp), "linear")
    h.dispose()
    if with_add:
        s = tf.add(T(shortcut), y)
        y.dispose()
        y = s
    if post == "relu":
        z = tf.relu(y)
        y.dispose()
        y = z
    elif post == "relu6":
        z = tf.relu6(y)
        y.dispose()
        y = z
    out = y.dataSync().reshape(y.shape)
    y.dispose()
    for t in made:
        t.dispose()
    return out


def _oracle(name, arrays):
    xs, n, dw_act, _, _, with_add, post, stride = _case(name)
    x, wd, bd, wp, bp, shortcut = arrays
    h = orc.fused_depthwise_conv2d(x, wd, stride, "same", bias=bd, activation=dw_act)
    y = orc.fused_conv2d(h, wp, 1, "same", bias=bp, activation="linear")
    if with_add:
        y = orc.binary("add", shortcut, y)
    if post:
        y = orc.unary(post, y)
    return y


@pytest.fixture
def every_shape(monkeypatch):
    """By default the library leaves large stride-1 maps to the two separate kernels (they
    are faster there); the parity cases run every tile shape of the fused kernel."""
    monkeypatch.setenv("TFJS_CUDA_DW_PROJECT_ALL", "1")


@pytest.mark.parametrize("name", sorted(CASES))
def test_folded_matches_separate_kernels_and_oracle(cuda_engine, every_shape, name):
    from tfjs_b200 import ops as tf
    arrays = _inputs(name)
    backend = cuda_engine.backend
    assert backend.lazy_fusion and backend.fuse_depthwise_project
    backend.launch_log(True)
    backend.launch_log_take()
    before = backend.launch_count()
    folded = _block(tf, name, arrays)
    launches = backend.launch_count() - before
    log = backend.launch_log_take()
    backend.launch_log(False)
    assert "dw_project_kernel" in log, log
    backend.fuse_depthwise_project = False
    try:
        before = backend.launch_count()
        separate = _block(tf, name, arrays)
        separate_launches = backend.launch_count() - before
    finally:
        backend.fuse_depthwise_project = True
    assert launches == separate_launches - 1
    assert np.array_equal(folded.view(np.uint32), separate.view(np.uint32)), \
        float(np.max(np.abs(folded - separate)))
    ref = _oracle(name, arrays)
    err = np.max(np.abs(folded.astype(np.float64) - ref)) / np.max(np.abs(ref))
    assert err <= TF32_TOL, err


def test_nan_follows_the_reference(cuda_engine, every_shape):
    """A NaN in the input reaches exactly the outputs whose 3x3 window holds it (every
    channel of them, through the projection), as in the reference."""
    from tfjs_b200 import ops as tf
    name = "linear_dw_no_bias"
    x, wd, bd, wp, bp, shortcut = _inputs(name)
    x = x.copy()
    x[1, 5, 7, 3] = np.nan
    arrays = (x, wd, bd, wp, bp, shortcut)
    got = _block(tf, name, arrays)
    ref = _oracle(name, arrays)
    assert np.array_equal(np.isnan(got), np.isnan(ref))
    assert np.isnan(got[1, 4:7, 6:9, :]).all() and not np.isnan(got[0]).any()
    ok = ~np.isnan(ref)
    assert np.max(np.abs(got[ok] - ref[ok])) <= TF32_TOL * np.max(np.abs(ref[ok]))


def test_unsupported_shapes_fall_back_to_two_launches(cuda_engine):
    """A dilated depthwise convolution is not taken by the fused kernel: the host layer
    launches the kernels separately and the result stands."""
    from tfjs_b200 import ops as tf
    r = np.random.default_rng(5)
    x = r.standard_normal((2, 15, 15, 32)).astype(np.float32)
    wd = (r.standard_normal((3, 3, 32, 1)) / 3).astype(np.float32)
    wp = (r.standard_normal((1, 1, 32, 16)) / 6).astype(np.float32)
    backend = cuda_engine.backend
    backend.launch_log(True)
    backend.launch_log_take()
    xt, wdt, wpt = tf.tensor(x), tf.tensor(wd), tf.tensor(wp)
    h = tf.fused_depthwise_conv2d(xt, wdt, 1, "same", "NHWC", [2, 2], None, None, "relu6")
    y = tf.fused_conv2d(h, wpt, 1, "same", "NHWC", [1, 1], None, None, "linear")
    got = y.dataSync().reshape(y.shape)
    log = backend.launch_log_take()
    backend.launch_log(False)
    for t in (xt, wdt, wpt, h, y):
        t.dispose()
    assert "dw_project_kernel" not in log
    ref = orc.fused_conv2d(orc.fused_depthwise_conv2d(x, wd, 1, "same", dilations=2,
                                                      activation="relu6"), wp, 1, "same")
    assert np.max(np.abs(got - ref)) <= TF32_TOL * np.max(np.abs(ref))


def test_shapes_the_kernel_declines_run_as_two_launches(cuda_engine):
    """Large stride-1 maps (the default choice) and projections too wide for the tile's
    shared memory are declined by the library; the two kernels run and the result stands."""
    from tfjs_b200 import ops as tf
    backend = cuda_engine.backend
    for name, xs, n in (("large_map", (1, 56, 56, 32), 16), ("wide_projection", (1, 20, 20, 32), 512)):
        r = np.random.default_rng(11)
        x = r.standard_normal(xs).astype(np.float32)
        wd = (r.standard_normal((3, 3, xs[3], 1)) / 3).astype(np.float32)
        wp = (r.standard_normal((1, 1, xs[3], n)) / 6).astype(np.float32)
        backend.launch_log(True)
        backend.launch_log_take()
        xt, wdt, wpt = tf.tensor(x), tf.tensor(wd), tf.tensor(wp)
        h = tf.fused_depthwise_conv2d(xt, wdt, 1, "same", "NHWC", [1, 1], None, None, "relu6")
        y = tf.fused_conv2d(h, wpt, 1, "same", "NHWC", [1, 1], None, None, "linear")
        got = y.dataSync().reshape(y.shape)
        log = backend.launch_log_take()
        backend.launch_log(False)
        for t in (xt, wdt, wpt, h, y):
            t.dispose()
        assert "dw_project_kernel" not in log, name
        ref = orc.fused_conv2d(orc.fused_depthwise_conv2d(x, wd, 1, "same", activation="relu6"),
                               wp, 1, "same")
        assert np.max(np.abs(got - ref)) <= TF32_TOL * np.max(np.abs(ref)), name


def test_depthwise_result_read_by_two_consumers(cuda_engine):
    """When the depthwise result is also read directly it materialises for that reader and
    the projection still gets the same values."""
    from tfjs_b200 import ops as tf
    r = np.random.default_rng(6)
    x = r.standard_normal((2, 14, 14, 64)).astype(np.float32)
    wd = (r.standard_normal((3, 3, 64, 1)) / 3).astype(np.float32)
    wp = (r.standard_normal((1, 1, 64, 24)) / 8).astype(np.float32)
    xt, wdt, wpt = tf.tensor(x), tf.tensor(wd), tf.tensor(wp)
    before = cuda_engine.backend.numDataIds()
    h = tf.fused_depthwise_conv2d(xt, wdt, 1, "same", "NHWC", [1, 1], None, None, "relu6")
    y = tf.fused_conv2d(h, wpt, 1, "same", "NHWC", [1, 1], None, None, "linear")
    hv = h.dataSync().reshape(h.shape)
    yv = y.dataSync().reshape(y.shape)
    h.dispose()
    y.dispose()
    assert cuda_engine.backend.numDataIds() == before
    for t in (xt, wdt, wpt):
        t.dispose()
    href = orc.fused_depthwise_conv2d(x, wd, 1, "same", activation="relu6")
    assert np.max(np.abs(hv - href)) <= 1e-6 * np.max(np.abs(href))
    yref = orc.fused_conv2d(href, wp, 1, "same")
    assert np.max(np.abs(yv - yref)) <= TF32_TOL * np.max(np.abs(yref))
