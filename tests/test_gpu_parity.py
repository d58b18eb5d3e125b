"""CUDA kernels vs the CPU oracle on the same seeded inputs (B200 only).

Tolerances: integer / indexing / copy kernels and the single-rounding fp32
elementwise kernels are bit-exact; tensor-core kernels (TF32 inputs, fp32
accumulation) must satisfy max|err| <= 2e-3 * max|ref|; the fp32 SIMT math mode
must satisfy max|err| <= 2e-5 * max|ref|.
"""
import numpy as np
import pytest

from oracle import oracle as orc
from tests import opcases

pytestmark = pytest.mark.gpu

TF32_TOL = 2e-3
FP32_TOL = 2e-5


def rel_err(got, ref):
    ref = np.asarray(ref, np.float64)
    got = np.asarray(got, np.float64)
    assert got.shape == ref.shape, (got.shape, ref.shape)
    denom = np.max(np.abs(ref)) if ref.size else 1.0
    return float(np.max(np.abs(got - ref)) / (denom if denom > 0 else 1.0)) if ref.size else 0.0


def rng(seed):
    return np.random.default_rng(seed)


def f32(a):
    return np.asarray(a, np.float32)


# ------------------------------------------------------------------ conv2d --
def conv_case(seed, xs, fs, strides=1, pad="same", dilations=1, bias=True, act="relu",
              prelu=None, alpha=None, rounding=None):
    r = rng(seed)
    fan_in = fs[0] * fs[1] * fs[2]
    inputs = {"x": f32(r.standard_normal(xs)),
              "filter": f32(r.standard_normal(fs) * np.sqrt(2.0 / fan_in))}
    if bias:
        inputs["bias"] = f32(r.standard_normal(fs[3]) * 0.1)
    if act == "prelu":
        inputs["preluActivationWeights"] = f32(
            r.standard_normal(fs[3] if prelu == "channel" else 1) * 0.3)
    return {"op": "fused_conv2d", "inputs": inputs,
            "attrs": {"strides": strides, "pad": pad, "dilations": dilations,
                      "activation": act, "leakyreluAlpha": alpha, "dimRoundingMode": rounding}}


CONV_CASES = {
    # BASELINE config 1: x[8,56,56,64], f[3,3,64,64], stride 1, same, relu, seed 0
    "cfg1": lambda: conv_case(0, (8, 56, 56, 64), (3, 3, 64, 64)),
    "3x3_s2_same": lambda: conv_case(1, (2, 28, 28, 128), (3, 3, 128, 128), strides=2),
    "3x3_cin32_cout24_tailN": lambda: conv_case(2, (3, 17, 19, 32), (3, 3, 32, 24), act="relu6"),
    "3x3_cin16_padK": lambda: conv_case(3, (2, 15, 15, 16), (3, 3, 16, 40), act="linear"),
    "3x3_cin48_padK": lambda: conv_case(4, (1, 14, 14, 48), (3, 3, 48, 64), act="elu"),
    "stem_7x7_s2_cin3": lambda: conv_case(5, (2, 64, 64, 3), (7, 7, 3, 64), strides=2),
    "stem_3x3_s2_cin3": lambda: conv_case(6, (2, 32, 32, 3), (3, 3, 3, 32), strides=2, act="relu6"),
    "1x1_pointwise": lambda: conv_case(7, (4, 14, 14, 96), (1, 1, 96, 576), act="relu6"),
    "1x1_k24": lambda: conv_case(8, (2, 28, 28, 24), (1, 1, 24, 144), act="relu6"),
    "1x1_cout1000": lambda: conv_case(9, (5, 1, 1, 1280), (1, 1, 1280, 1000), act="linear"),
    "1x1_s2_projection": lambda: conv_case(10, (2, 28, 28, 64), (1, 1, 64, 128), strides=2, pad="same", act="linear"),
    "dilation2": lambda: conv_case(11, (1, 20, 20, 32), (3, 3, 32, 32), dilations=2, act="sigmoid"),
    "valid_pad": lambda: conv_case(12, (2, 13, 13, 64), (3, 3, 64, 64), pad="valid", act="leakyrelu", alpha=0.3),
    "explicit_pad": lambda: conv_case(13, (1, 9, 9, 32), (3, 3, 32, 16), pad=[[0, 0], [1, 2], [0, 1], [0, 0]], act="prelu", prelu="channel"),
    "prelu_scalar_nobias": lambda: conv_case(14, (1, 8, 8, 32), (3, 3, 32, 32), bias=False, act="prelu", prelu="scalar"),
    "wide_cout256": lambda: conv_case(15, (2, 14, 14, 256), (3, 3, 256, 256)),
    "cin5_simt_route": lambda: conv_case(16, (1, 9, 9, 5), (2, 2, 5, 7), pad="valid"),
    # 3 x 3 on a 3-channel image: the fp32 SIMT stem kernel (both math modes)
    "stem_3x3_s1_cout8_valid": lambda: conv_case(22, (2, 19, 23, 3), (3, 3, 3, 8), pad="valid", act="linear"),
    "stem_3x3_s2_cout64_prelu": lambda: conv_case(23, (1, 30, 30, 3), (3, 3, 3, 64), strides=2, act="prelu", prelu="channel"),
    "stem_3x3_s2_224_cout32": lambda: conv_case(24, (1, 224, 224, 3), (3, 3, 3, 32), strides=2, act="relu6"),
    "stem_3x3_s1_explicit_pad_cout16": lambda: conv_case(25, (2, 9, 70, 3), (3, 3, 3, 16), pad=[[0, 0], [2, 1], [0, 3], [0, 0]], bias=False, act="sigmoid"),
    # 14 tiles of 144 K steps (ResNet conv5 at a small batch): K-split over all SMs
    "k_split_conv5": lambda: conv_case(21, (16, 7, 7, 512), (3, 3, 512, 512)),
    # long K, <= 128 output channels: the form with the pixels on the MMA's N axis
    "narrow_1x1_k416_cout100": lambda: conv_case(17, (3, 10, 11, 416), (1, 1, 416, 100), act="linear"),
    "narrow_3x3_cout96_ragged": lambda: conv_case(18, (3, 21, 23, 64), (3, 3, 64, 96), act="relu6"),
    "narrow_dilated_nobias": lambda: conv_case(19, (1, 20, 20, 64), (3, 3, 64, 32), dilations=2, bias=False, act="sigmoid"),
    "narrow_s2_valid_cout4": lambda: conv_case(20, (2, 15, 15, 128), (3, 3, 128, 4), strides=2, pad="valid"),
}


@pytest.mark.parametrize("name", sorted(CONV_CASES))
@pytest.mark.parametrize("mode", ["tf32", "fp32"])
def test_fused_conv2d(cuda_engine, name, mode):
    case = CONV_CASES[name]()
    ref = opcases.run_oracle(case)
    cuda_engine.backend.set_math_mode(mode)
    try:
        got = opcases.run_cuda(case)
    finally:
        cuda_engine.backend.set_math_mode("tf32")
    err = rel_err(got, ref)
    assert err <= (TF32_TOL if mode == "tf32" else FP32_TOL), (name, mode, err)


def test_conv2d_bias_broadcast_unfused(cuda_engine):
    """A bias that is not per-channel goes through the separate Add kernel."""
    case = conv_case(20, (1, 6, 6, 8), (3, 3, 8, 8))
    case["inputs"]["bias"] = f32(rng(21).standard_normal((6, 6, 8)))
    err = rel_err(opcases.run_cuda(case), opcases.run_oracle(case))
    assert err <= TF32_TOL


# ------------------------------------------------------------------ matmul --
def mm_case(seed, a_shape, b_shape, ta=False, tb=False, bias=None, act="linear", scale=None):
    r = rng(seed)
    k = a_shape[-2] if ta else a_shape[-1]
    s = scale if scale is not None else 1.0 / np.sqrt(max(k, 1))
    inputs = {"a": f32(r.standard_normal(a_shape) * s), "b": f32(r.standard_normal(b_shape) * s)}
    n = b_shape[-2] if tb else b_shape[-1]
    op = "mat_mul"
    attrs = {"transposeA": ta, "transposeB": tb}
    if bias is not None or act != "linear":
        op = "fused_mat_mul"
        if bias:
            inputs["bias"] = f32(r.standard_normal(n) * 0.1)
        attrs["activation"] = act
    return {"op": op, "inputs": inputs, "attrs": attrs}


MM_CASES = {
    # BASELINE config 2b: a[32,512,64] x b[32,64,512] ~ N(0,1)
    "cfg2b": lambda: mm_case(0, (32, 512, 64), (32, 64, 512), scale=1.0),
    "dense_1280_1000": lambda: mm_case(1, (64, 1280), (1280, 1000), bias=True),
    "ffn_768_3072": lambda: mm_case(2, (256, 768), (768, 3072), bias=True, act="relu6"),
    "attn_qk": lambda: mm_case(3, (24, 128, 64), (24, 128, 64), tb=True, scale=0.5),
    "attn_pv": lambda: mm_case(4, (24, 128, 128), (24, 128, 64), scale=0.2),
    "bcast_b": lambda: mm_case(5, (6, 70, 36), (1, 36, 52)),
    "bcast_a": lambda: mm_case(6, (1, 33, 40), (5, 40, 20)),
    "rank4": lambda: mm_case(7, (2, 3, 50, 32), (2, 3, 32, 44)),
    "transpose_a": lambda: mm_case(8, (2, 48, 70), (2, 48, 36), ta=True),
    "transpose_ab": lambda: mm_case(9, (64, 30), (50, 64), ta=True, tb=True),
    "k_not_mult4": lambda: mm_case(10, (37, 13), (13, 29), bias=True, act="elu"),
    "k1000_n10": lambda: mm_case(11, (130, 1000), (1000, 10), bias=True, act="sigmoid"),
    "tall_m": lambda: mm_case(12, (3000, 64), (64, 96), act="relu"),
    # 10 tiles with 128 K steps each: the K steps are shared out over all SMs and every
    # tile is summed from the partial tiles of about 15 CTAs
    "k_split_long_k": lambda: mm_case(13, (640, 4096), (4096, 512), bias=True, act="relu"),
    # one full wave of tiles and a remainder of 30 whose K steps are split (178 tiles)
    "k_split_tail_wave": lambda: mm_case(14, (11392, 1536), (1536, 512), bias=True),
}


@pytest.mark.parametrize("name", sorted(MM_CASES))
@pytest.mark.parametrize("mode", ["tf32", "fp32"])
def test_matmul(cuda_engine, name, mode):
    case = MM_CASES[name]()
    ref = opcases.run_oracle(case)
    cuda_engine.backend.set_math_mode(mode)
    try:
        got = opcases.run_cuda(case)
    finally:
        cuda_engine.backend.set_math_mode("tf32")
    err = rel_err(got, ref)
    assert err <= (TF32_TOL if mode == "tf32" else FP32_TOL), (name, mode, err)


@pytest.mark.parametrize("name", ["cfg2b", "attn_pv", "attn_qk", "bcast_b", "rank4", "tall_m",
                                  "dense_1280_1000", "k1000_n10"])
def test_matmul_activation_b(cuda_engine, name):
    """B produced on the device (an activation, not a weight): the tensor-core
    kernel streams it as stored, MN-major or K-major, instead of a packed copy."""
    case = dict(MM_CASES[name](), device_inputs=["b"])
    err = rel_err(opcases.run_cuda(case), opcases.run_oracle(case))
    assert err <= TF32_TOL, (name, err)


def test_fused_matmul_cfg2a_rows(cuda_engine):
    """BASELINE config 2a at full size on the GPU; the oracle checks a sample of
    rows (every row of the product depends on one row of A only)."""
    r = rng(0)
    s = 1.0 / np.sqrt(1024)
    a = f32(r.standard_normal((4096, 1024)) * s)
    b = f32(r.standard_normal((1024, 4096)) * s)
    bias = f32(r.standard_normal(4096) * 0.1)
    case = {"op": "fused_mat_mul", "inputs": {"a": a, "b": b, "bias": bias},
            "attrs": {"activation": "relu6"}}
    got = opcases.run_cuda(case)
    rows = np.concatenate([np.arange(0, 4096, 61), [127, 128, 4095]])
    ref = orc.fused_matmul(a[rows], b, bias=bias, activation="relu6")
    assert rel_err(got[rows], ref) <= TF32_TOL
    # weights were packed once; a second call reuses the packed copy
    got2 = opcases.run_cuda(case)
    assert np.array_equal(got, got2)


def test_k_split_matmul_is_deterministic(cuda_engine):
    """Partial tiles are added in CTA order, so two launches give the same bits."""
    case = MM_CASES["k_split_long_k"]()
    a, b = opcases.run_cuda(case), opcases.run_cuda(case)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


def test_matmul_nan_propagates(cuda_engine):
    a = f32([[1, 2, np.nan, 4], [5, 6, 7, 8]])
    b = f32(np.ones((4, 4)))
    for mode in ("tf32", "fp32"):
        cuda_engine.backend.set_math_mode(mode)
        got = opcases.run_cuda({"op": "mat_mul", "inputs": {"a": a, "b": b}})
        cuda_engine.backend.set_math_mode("tf32")
        assert np.isnan(got[0]).all() and np.array_equal(got[1], f32([26] * 4))


def test_matmul_zero_sized(cuda_engine):
    got = opcases.run_cuda({"op": "mat_mul", "inputs": {"a": np.zeros((3, 0), np.float32),
                                                        "b": np.zeros((0, 2), np.float32)}})
    assert got.shape == (3, 2) and np.array_equal(got, np.zeros((3, 2), np.float32))
    got = opcases.run_cuda({"op": "mat_mul", "inputs": {"a": np.zeros((0, 3), np.float32),
                                                        "b": np.zeros((3, 2), np.float32)}})
    assert got.shape == (0, 2)


# --------------------------------------------------------------- depthwise --
def dw_case(seed, xs, fs, strides=1, pad="same", dilations=1, bias=True, act="relu6"):
    r = rng(seed)
    inputs = {"x": f32(r.standard_normal(xs)),
              "filter": f32(r.standard_normal(fs) * np.sqrt(2.0 / (fs[0] * fs[1])))}
    if bias:
        inputs["bias"] = f32(r.standard_normal(fs[2] * fs[3]) * 0.1)
    if act == "prelu":
        inputs["preluActivationWeights"] = f32(r.standard_normal(fs[2] * fs[3]) * 0.3)
    return {"op": "fused_depthwise_conv2d", "inputs": inputs,
            "attrs": {"strides": strides, "pad": pad, "dilations": dilations, "activation": act}}


DW_CASES = {
    "mbv2_112_c32_s1": lambda: dw_case(0, (2, 112, 112, 32), (3, 3, 32, 1)),
    "mbv2_112_c96_s2": lambda: dw_case(1, (2, 112, 112, 96), (3, 3, 96, 1), strides=2),
    "mbv2_7_c960": lambda: dw_case(2, (4, 7, 7, 960), (3, 3, 960, 1)),
    # widths that are multiples of 28 take 28-wide tiles with seven outputs per thread
    "mbv2_56_c144_s1": lambda: dw_case(7, (2, 56, 56, 144), (3, 3, 144, 1)),
    "w28_c40_h13_valid": lambda: dw_case(8, (3, 15, 30, 40), (3, 3, 40, 1), pad="valid", act="relu"),
    "w84_c8": lambda: dw_case(9, (1, 20, 84, 8), (3, 3, 8, 1), act="linear", bias=False),
    "chmul2": lambda: dw_case(3, (2, 9, 11, 6), (3, 3, 6, 2), act="relu"),
    "c5_scalar_path": lambda: dw_case(4, (1, 10, 10, 5), (3, 3, 5, 1), pad="valid", act="elu"),
    "dilated": lambda: dw_case(5, (1, 16, 16, 8), (3, 3, 8, 1), dilations=2, act="linear", bias=False),
    "prelu": lambda: dw_case(6, (1, 8, 8, 16), (3, 3, 16, 1), act="prelu"),
}


@pytest.mark.parametrize("name", sorted(DW_CASES))
def test_fused_depthwise(cuda_engine, name):
    case = DW_CASES[name]()
    err = rel_err(opcases.run_cuda(case), opcases.run_oracle(case))
    assert err <= 1e-6, (name, err)


# ------------------------------------------------------------------- pools --
@pytest.mark.parametrize("kind", ["max_pool", "avg_pool"])
@pytest.mark.parametrize("cfg", [((2, 112, 112, 64), 3, 2, "same"), ((1, 9, 9, 5), 2, 1, "valid"),
                                 ((2, 7, 7, 32), 7, 1, "valid"), ((1, 8, 8, 4), 3, 1, 1),
                                 # 3x3 stride 2 with channels % 4 == 0: the four-column max kernel
                                 ((3, 15, 13, 8), 3, 2, "valid"), ((2, 9, 10, 4), 3, 2, "same"),
                                 ((1, 12, 21, 12), 3, 2, 1)])
def test_pool(cuda_engine, kind, cfg):
    shape, fsz, stride, pad = cfg
    x = f32(rng(3).standard_normal(shape))
    case = {"op": kind, "inputs": {"x": x}, "attrs": {"filterSize": fsz, "strides": stride, "pad": pad}}
    got, ref = opcases.run_cuda(case), opcases.run_oracle(case)
    assert np.array_equal(got, ref), rel_err(got, ref)


def test_maxpool_ignores_nan(cuda_engine):
    x = f32(rng(4).standard_normal((1, 6, 6, 4)))
    x[0, 2, 2, 1] = np.nan
    case = {"op": "max_pool", "inputs": {"x": x}, "attrs": {"filterSize": 2, "strides": 2, "pad": "valid"}}
    assert np.array_equal(opcases.run_cuda(case), opcases.run_oracle(case), equal_nan=True)


def test_maxpool3x3s2_ignores_nan_and_handles_all_nan_windows(cuda_engine):
    x = f32(rng(5).standard_normal((2, 11, 14, 8)))
    x[0, 4, 6, 3] = np.nan
    x[1, 0:3, 0:3, 5] = np.nan          # a whole window: the result stays -inf, as in the reference
    case = {"op": "max_pool", "inputs": {"x": x}, "attrs": {"filterSize": 3, "strides": 2, "pad": "valid"}}
    assert np.array_equal(opcases.run_cuda(case), opcases.run_oracle(case), equal_nan=True)


# -------------------------------------------------------------- elementwise --
EXACT_UNARY = ["relu", "relu6", "sqrt", "square", "neg", "abs"]
DOUBLE_UNARY = ["elu", "sigmoid", "exp", "rsqrt", "tanh", "erf", "log"]


def _in_mode(engine, mode, case):
    """Runs a case with the backend in math mode 'fp32' (the reference's double-precision
    evaluation order, fp32 store) or 'tf32' (the default: fp32 evaluations of exp / erf /
    tanh and an fp32 softmax sum)."""
    engine.backend.set_math_mode(mode)
    try:
        return opcases.run_cuda(case)
    finally:
        engine.backend.set_math_mode("tf32")


# Bounds of the default mode's fp32 evaluations against the double-precision oracle: a few
# units in the last place for exp / sigmoid / tanh / elu; erf is the reference's polynomial
# in fp32 with the special-function unit's reciprocal and exponential (1 and 2 units in the
# last place), whose cancellation near zero leaves an absolute error.
FP32_EVAL_REL = 6e-7
FP32_ERF_ABS = 8e-7


@pytest.mark.parametrize("mode", ["fp32", "tf32"])
@pytest.mark.parametrize("op", EXACT_UNARY + DOUBLE_UNARY)
def test_unary(cuda_engine, op, mode):
    x = f32(rng(5).standard_normal(100003) * 3)
    if op in ("sqrt", "rsqrt", "log"):
        x = np.abs(x) + 1e-3
    x[:4] = [np.nan, 0.0, -0.0, np.inf]
    case = {"op": op, "inputs": {"x": x}}
    got, ref = _in_mode(cuda_engine, mode, case), opcases.run_oracle(case)
    if op in EXACT_UNARY:
        assert np.array_equal(got, ref, equal_nan=True)
    else:
        ok = np.isfinite(ref)
        assert np.array_equal(np.isnan(got), np.isnan(ref))
        if mode == "tf32" and op == "erf":
            assert np.max(np.abs(got[ok] - ref[ok])) <= FP32_ERF_ABS
            return
        # fp32 mode: device and host libm may differ in the last bit of the double result
        bound = 2.5e-7 if mode == "fp32" else FP32_EVAL_REL
        assert np.max(np.abs(got[ok] - ref[ok]) / np.maximum(np.abs(ref[ok]), 1e-30)) <= bound


@pytest.mark.parametrize("mode", ["fp32", "tf32"])
@pytest.mark.parametrize("op", ["erf", "exp", "sigmoid"])
def test_unary_wide_range(cuda_engine, op, mode):
    """Magnitudes from 1e-9 to beyond the range where exp over- or underflows.  fp32 mode:
    the device evaluates erf and exp with a shortened double sequence except near zero
    (erf) and beyond +-700 (exp).  tf32 mode: fp32 evaluations; results below the smallest
    normal fp32 number may flush to zero."""
    r = rng(55)
    mag = 10.0 ** r.uniform(-9, 1.6 if op == "erf" else 2.0, 200000)
    x = f32(mag * np.where(r.random(200000) < 0.5, -1.0, 1.0))
    x[:8] = [np.nan, 0.0, -0.0, np.inf, -np.inf, 2.0 ** -13, -2.0 ** -13, 88.0]
    case = {"op": op, "inputs": {"x": x}}
    with np.errstate(over="ignore"):
        got, ref = _in_mode(cuda_engine, mode, case), opcases.run_oracle(case)
    assert np.array_equal(np.isnan(got), np.isnan(ref))
    ok = np.isfinite(ref)
    if mode == "tf32":
        err = np.abs(got[ok].astype(np.float64) - ref[ok])
        if op == "erf":
            assert np.max(err) <= FP32_ERF_ABS
            assert np.array_equal(np.signbit(got[ok]), np.signbit(ref[ok]))
        else:
            # relative, with an absolute floor near the fp32 normal limit (sigmoid of a very
            # negative argument is the reciprocal of a number close to the largest float, a
            # subnormal with few bits); an overflow to infinity may come one ulp of the
            # argument early or late
            assert np.max(err[np.isfinite(got[ok])] /
                          (np.abs(ref[ok][np.isfinite(got[ok])]) + 1e-32)) <= FP32_EVAL_REL
            assert np.all(np.abs(ref[ok][np.isinf(got[ok])]) > 3e38)
        return
    assert np.array_equal(np.isinf(got), np.isinf(ref))
    assert np.array_equal(np.signbit(got[ok]), np.signbit(ref[ok]))
    assert np.max(np.abs(got[ok] - ref[ok]) / np.maximum(np.abs(ref[ok]), 1e-37)) <= 2.5e-7
    # the shortened sequence changes the rounding of very few results
    assert np.mean(got[ok] != ref[ok]) < 1e-3


def test_leakyrelu_clip(cuda_engine):
    x = f32(rng(6).standard_normal(5000) * 4)
    for case in ({"op": "leaky_relu", "inputs": {"x": x}, "attrs": {"alpha": 0.2}},
                 {"op": "clip_by_value", "inputs": {"x": x}, "attrs": {"lo": -1.5, "hi": 2.25}}):
        assert np.array_equal(opcases.run_cuda(case), opcases.run_oracle(case))


BIN_SHAPES = [((4, 56, 56, 64), (4, 56, 56, 64)), ((8, 49, 320), (320,)), ((320,), (8, 49, 320)),
              ((7, 5, 3), (1,)), ((3, 1, 5), (1, 4, 1)), ((2, 3, 4, 5), (4, 1)), ((6,), ()),
              # attention mask against scores: equal on the outer and inner axes, 1 in between
              ((4, 12, 128, 128), (4, 1, 1, 128)), ((3, 1, 1, 64), (3, 5, 7, 64)),
              ((2, 6, 8), (2, 1, 8)), ((5, 3, 2, 4, 12), (5, 3, 1, 1, 12)),
              # periods that do not divide the grid stride
              ((1000, 772), (772,)), ((33, 7, 20), (7, 20))]


@pytest.mark.parametrize("op", ["add", "sub", "mul", "div", "maximum", "minimum",
                                "squared_difference", "pow"])
@pytest.mark.parametrize("shapes", BIN_SHAPES)
def test_binary(cuda_engine, op, shapes):
    r = rng(7)
    a = f32(r.standard_normal(shapes[0]))
    b = f32(r.standard_normal(shapes[1]))
    if op == "pow":
        a = np.abs(a) + 0.1
    case = {"op": op, "inputs": {"a": a, "b": b}}
    got, ref = opcases.run_cuda(case), opcases.run_oracle(case)
    if op == "pow":
        assert rel_err(got, ref) <= 1e-6
    else:
        assert np.array_equal(got, ref, equal_nan=True)


def test_binary_int32(cuda_engine):
    r = rng(8)
    a = r.integers(-1000, 1000, (5, 7)).astype(np.int32)
    b = r.integers(1, 50, (7,)).astype(np.int32)
    for op in ("add", "sub", "mul", "maximum", "minimum"):
        case = {"op": op, "inputs": {"a": a, "b": b}}
        got = opcases.run_cuda(case)
        assert got.dtype == np.int32 and np.array_equal(got, opcases.run_oracle(case))


def test_prelu_and_batchnorm(cuda_engine):
    r = rng(9)
    x = f32(r.standard_normal((4, 6, 8)))
    case = {"op": "prelu", "inputs": {"x": x, "alpha": f32(r.standard_normal(8))}}
    assert np.array_equal(opcases.run_cuda(case), opcases.run_oracle(case))
    case = {"op": "batch_norm",
            "inputs": {"x": x, "mean": f32(r.standard_normal(8)),
                       "variance": f32(np.abs(r.standard_normal(8)) + 0.1),
                       "offset": f32(r.standard_normal(8)), "scale": f32(r.standard_normal(8))},
            "attrs": {"varianceEpsilon": 1e-3}}
    assert rel_err(opcases.run_cuda(case), opcases.run_oracle(case)) <= 3e-7


# --------------------------------------------------------------- reductions --
@pytest.mark.parametrize("shape", [(64, 12, 16, 128), (70, 1000), (3, 2500), (5, 1)])
@pytest.mark.parametrize("mode", ["fp32", "tf32"])
def test_softmax(cuda_engine, shape, mode):
    x = f32(rng(10).standard_normal(shape) * 4)
    case = {"op": "softmax", "inputs": {"logits": x}}
    got, ref = _in_mode(cuda_engine, mode, case), opcases.run_oracle(case)
    # fp32 mode: double sum as the reference; tf32 mode: expf and an fp32 sum
    bound = 1.5e-7 if mode == "fp32" else 1e-6
    assert np.max(np.abs(got - ref)) <= bound, np.max(np.abs(got - ref))


@pytest.mark.parametrize("op", ["sum", "mean", "max"])
@pytest.mark.parametrize("cfg", [((8, 7, 7, 1280), [1, 2], False), ((64, 128, 768), -1, True),
                                 ((6, 5, 4, 3), [0, 2], False), ((10, 11), None, False),
                                 ((3, 4, 5), 0, True)])
def test_reduce(cuda_engine, op, cfg):
    shape, axis, keep = cfg
    x = f32(rng(11).standard_normal(shape))
    case = {"op": op, "inputs": {"x": x}, "attrs": {"axis": axis, "keepDims": keep}}
    got, ref = opcases.run_cuda(case), opcases.run_oracle(case)
    assert got.shape == ref.shape
    if op == "max":
        assert np.array_equal(got, ref)
    else:
        assert np.max(np.abs(got - ref) / np.maximum(np.abs(ref), 1e-6)) <= 1.5e-7


def test_argmax_bit_exact(cuda_engine):
    r = rng(12)
    x = f32(r.standard_normal((300, 1000)))
    x[5, 10] = x[5, 900] = 50.0       # tie -> first index
    x[6, 0] = np.nan                  # NaN first -> 0
    x[7, 500] = np.nan                # NaN elsewhere is skipped
    for axis, arr in ((1, x), (0, x[:64]), (1, f32(r.standard_normal((4, 5, 6))))):
        case = {"op": "arg_max", "inputs": {"x": arr}, "attrs": {"axis": axis}}
        got = opcases.run_cuda(case)
        assert got.dtype == np.int32 and np.array_equal(got, opcases.run_oracle(case))


# ----------------------------------------------------------------- movement --
@pytest.mark.parametrize("cfg", [((64, 128, 12, 64), [0, 2, 1, 3]), ((5, 7), [1, 0]),
                                 ((3, 40, 50), [0, 2, 1]), ((2, 3, 4, 5), [3, 1, 0, 2]),
                                 ((2, 1, 6, 4), [0, 2, 1, 3]), ((4, 6), [0, 1])])
def test_transpose(cuda_engine, cfg):
    shape, perm = cfg
    x = f32(rng(13).standard_normal(shape))
    case = {"op": "transpose", "inputs": {"x": x}, "attrs": {"perm": perm}}
    assert np.array_equal(opcases.run_cuda(case), opcases.run_oracle(case))


def test_gather_bit_exact_and_range_check(cuda_engine):
    r = rng(14)
    table = f32(r.standard_normal((30522, 768)))
    ids = r.integers(0, 30522, (64, 128)).astype(np.int32)
    case = {"op": "gather", "inputs": {"x": table, "indices": ids}, "attrs": {"axis": 0}}
    assert np.array_equal(opcases.run_cuda(case), opcases.run_oracle(case))
    x = f32(r.standard_normal((3, 5, 7)))
    idx = np.array([[4, 0], [1, 1]], np.int32)
    case = {"op": "gather", "inputs": {"x": x, "indices": idx}, "attrs": {"axis": 1}}
    assert np.array_equal(opcases.run_cuda(case), opcases.run_oracle(case))
    for bad in (np.array([0, 5], np.int32), np.array([-1, 2], np.int32),
                np.full((40, 40), 9, np.int32)):   # host-resident and device-resident indices
        with pytest.raises(ValueError, match="is not in"):
            opcases.run_cuda({"op": "gather", "inputs": {"x": x, "indices": bad},
                              "attrs": {"axis": 1}})


def test_cast_js_semantics(cuda_engine):
    x = f32([1.9, -1.9, 0.5, -0.5, np.nan, np.inf, -np.inf, 3e9, -3e9, 2147483648.0, 1e20, 0.0])
    case = {"op": "cast", "inputs": {"x": x}, "attrs": {"dtype": "int32"}}
    got = opcases.run_cuda(case)
    assert got.dtype == np.int32 and np.array_equal(got, opcases.run_oracle(case))
    big = f32(rng(15).standard_normal(10000) * 1e3)
    case = {"op": "cast", "inputs": {"x": big}, "attrs": {"dtype": "int32"}}
    assert np.array_equal(opcases.run_cuda(case), opcases.run_oracle(case))
    case = {"op": "cast", "inputs": {"x": x}, "attrs": {"dtype": "bool"}}
    assert np.array_equal(opcases.run_cuda(case), opcases.run_oracle(case))
    ints = np.array([-3, 0, 7], np.int32)
    case = {"op": "cast", "inputs": {"x": ints}, "attrs": {"dtype": "float32"}}
    assert np.array_equal(opcases.run_cuda(case), f32([-3, 0, 7]))


def test_concat_slice_pad_tile(cuda_engine):
    r = rng(16)
    a, b, c = (f32(r.standard_normal(s)) for s in ((2, 3, 4), (2, 5, 4), (2, 1, 4)))
    for case in (
        {"op": "concat", "inputs": {"tensors": [a, b, c]}, "attrs": {"axis": 1}},
        {"op": "concat", "inputs": {"tensors": [a, a]}, "attrs": {"axis": -1}},
        {"op": "slice", "inputs": {"x": b}, "attrs": {"begin": [0, 1, 2], "size": [2, 3, -1]}},
        {"op": "slice", "inputs": {"x": b}, "attrs": {"begin": [1], "size": [1]}},
        {"op": "pad", "inputs": {"x": a}, "attrs": {"paddings": [[1, 0], [0, 2], [3, 1]], "constantValue": 1.5}},
        {"op": "tile", "inputs": {"x": c}, "attrs": {"reps": [2, 3, 1]}},
    ):
        assert np.array_equal(opcases.run_cuda(case), opcases.run_oracle(case)), case["op"]


# --------------------------------------------------------------- dequantise --
@pytest.mark.parametrize("qdtype", [np.uint8, np.uint16])
@pytest.mark.parametrize("target", ["float32", "int32"])
def test_dequantize_bit_exact(cuda_engine, qdtype, target):
    from tfjs_b200 import io
    r = rng(17)
    n = 100003
    q = r.integers(0, np.iinfo(qdtype).max + 1, n).astype(qdtype)
    scale, mn = 0.0123456789 * (256 if target == "int32" else 1), -1.57
    info = io.dequantize_to_device(cuda_engine.backend, q, scale, mn, [n], target)
    got = cuda_engine.backend.readSync(info.dataId)
    cuda_engine.backend.disposeData(info.dataId)
    ref = orc.dequantize(q, scale, mn, target)
    assert got.dtype == ref.dtype and np.array_equal(got, ref)


# ------------------------------------------------------------------ storage --
def test_storage_contract(cuda_engine):
    b = cuda_engine.backend
    n0 = b.numDataIds()
    small = b.write(np.arange(6, dtype=np.float32), [2, 3], "float32")
    assert b.host_values(small) is not None            # host-resident until used
    big_vals = np.arange(5000, dtype=np.float32)
    big = b.write(big_vals, [5000], "float32")
    assert b.host_values(big) is None
    assert b.numDataIds() == n0 + 2
    assert np.array_equal(b.readSync(big), big_vals)
    b.incRef(big)
    assert b.refCount(big) == 2
    assert b.disposeData(big) is False and b.numDataIds() == n0 + 2
    assert b.disposeData(big) is True and b.numDataIds() == n0 + 1
    assert b.disposeData(small, True) is True
    mem = b.memory()
    assert mem["unreliable"] is False and mem["numBytesInGPU"] >= 0
    from tfjs_b200.backend import CudaError
    with pytest.raises(CudaError):
        b.check(b.lib.tfjs_cuda_free(b.ctx, 999999))
    t = b.time(lambda: None)
    assert t["kernelMs"] >= 0.0


def test_reshape_is_zero_copy(cuda_engine):
    from tfjs_b200 import ops
    x = ops.tensor(np.arange(5000, dtype=np.float32), [50, 100], "float32")
    y = ops.reshape(x, [100, -1])
    assert y.dataId is x.dataId and y.shape == [100, 50]
    assert cuda_engine.backend.refCount(x.dataId) == 2
    x.dispose()
    assert np.array_equal(y.dataSync(), np.arange(5000, dtype=np.float32))
    y.dispose()


def test_missing_kernel_is_an_error(cuda_engine):
    with pytest.raises(RuntimeError, match="not registered for backend 'cuda'"):
        cuda_engine.run_kernel("NonMaxSuppressionV5", {}, {})


def test_overlapped_upload(cuda_engine):
    """tfjs_cuda_upload: copy-stream transfer; the first consumer waits for it."""
    from tfjs_b200 import ops
    from tfjs_b200.backend import TensorInfo
    b = cuda_engine.backend
    r = rng(30)
    big = b.pinned_empty((512, 1024), "float32")
    big[...] = r.standard_normal((512, 1024)).astype(np.float32)
    for _ in range(3):
        # keep the compute stream busy, then upload and consume right away
        busy = ops.tensor(np.ones((2048, 2048), np.float32))
        prod = ops.mat_mul(busy, busy)
        did = b.write_from(big, big.shape, "float32")
        t = cuda_engine.make_tensor_from_info(TensorInfo(did, big.shape, "float32"))
        doubled = ops.add(t, t)
        assert np.array_equal(doubled.arraySync(), big * 2)
        assert np.array_equal(t.dataSync().reshape(big.shape), big)
        for x in (busy, prod, t, doubled):
            x.dispose()
    # an uploaded tensor that is never consumed can still be freed
    did = b.write_from(big, big.shape, "float32")
    assert b.disposeData(did) is True
    b.sync()


def test_float16_weights_decode_on_device_bit_exact(cuda_engine):
    """Every half-precision bit pattern (NaN payloads included) and a ragged length,
    through decode_weights with a 'float16' quantised manifest entry."""
    from tfjs_b200 import io
    every = np.arange(65536, dtype=np.uint32).astype(np.uint16)
    r = rng(77)
    ragged = r.integers(0, 65536, 1003).astype(np.uint16)
    specs = [{"name": "every", "dtype": "float32", "shape": [256, 256],
              "quantization": {"dtype": "float16"}},
             {"name": "ragged", "dtype": "float32", "shape": [1003],
              "quantization": {"dtype": "float16"}},
             {"name": "empty", "dtype": "float32", "shape": [0],
              "quantization": {"dtype": "float16"}}]
    tensors = io.decode_weights(cuda_engine, every.tobytes() + ragged.tobytes(), specs)
    for name, src in (("every", every), ("ragged", ragged)):
        got = tensors[name].dataSync()
        ref = orc.decode_float16(src)
        assert np.array_equal(got.view(np.uint32), ref.view(np.uint32)), name
    assert tensors["empty"].shape == [0]
    for t in tensors.values():
        t.dispose()
