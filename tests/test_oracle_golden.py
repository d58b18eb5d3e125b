"""Pins the CPU oracle (and the host-side shape rules it shares with nothing)
against the reference's own known-answer vectors.  No GPU needed."""
import os

import numpy as np
import pytest

from oracle import oracle as orc
from tests import goldens, opcases

CASES, SUMMARY = goldens.load_ts_goldens()
TEST_EPSILON_FLOAT32 = 1e-3   # tfjs-core/src/test_util.ts:23


def test_fixture_covers_the_hot_path():
    assert len(CASES) >= 250
    ops = set(c["op"] for c in CASES)
    for needed in ("fused_conv2d", "fused_mat_mul", "fused_depthwise_conv2d", "mat_mul",
                   "conv2d", "depthwise_conv2d", "max_pool", "avg_pool", "softmax", "gather",
                   "arg_max", "mean", "sum", "max", "add", "relu", "erf", "transpose",
                   "batch_norm"):
        assert needed in ops, needed
    for rel in ("tfjs-core/src/ops/fused/fused_conv2d_test.ts",
                "tfjs-core/src/ops/fused/fused_mat_mul_test.ts",
                "tfjs-core/src/ops/mat_mul_test.ts"):
        assert SUMMARY[rel]["extracted_specs"] >= 15


@pytest.mark.parametrize("case", CASES, ids=[goldens.case_id(c) for c in CASES])
def test_oracle_matches_reference_vector(case):
    got = opcases.run_oracle(case)
    if case.get("squeeze0"):
        got = got[0]
    assert list(got.shape) == case["expected_shape"]
    ok, why = goldens.arrays_close(got, case["expected"], TEST_EPSILON_FLOAT32)
    assert ok, why


def test_quantization_fixtures():
    """oracle.dequantize and io.quantize_weights vs the reference's quantization.py."""
    from tfjs_b200 import io
    z = np.load(os.path.join(os.path.dirname(__file__), "golden", "quant_goldens.npz"))
    for key in z["names"]:
        data, q = z[key + "_data"], z[key + "_q"]
        mn, scale = float(z[key + "_min"]), float(z[key + "_scale"])
        q2, meta = io.quantize_weights(data, q.dtype)
        assert np.array_equal(q2, q), key
        assert float(meta["min"]) == mn and float(meta["scale"]) == scale, key
        deq = orc.dequantize(q, scale, mn, "float32")
        assert np.array_equal(deq, z[key + "_deq"]), key
    q = z["io_utils_q"]
    mn, scale = float(z["io_utils_min"]), float(z["io_utils_scale"])
    assert np.allclose(orc.dequantize(q, scale, mn, "float32"), z["io_utils_f32"], atol=1e-3)
    assert np.array_equal(orc.dequantize(q, scale, mn, "int32"), z["io_utils_i32"])
    assert np.array_equal(orc.dequantize(q.astype(np.uint16), scale, mn, "int32"),
                          z["io_utils_i32"])


def test_js_numerics_details():
    """Spot checks of the JavaScript rules the oracle restates."""
    nan = float("nan")
    x = np.array([nan, -0.0, 0.0, 7.0, -3.0], np.float32)
    r = orc.unary("relu", x)
    assert np.isnan(r[0]) and not np.signbit(r[1]) and r[3] == 7 and r[4] == 0
    assert np.isnan(orc.unary("relu6", x)[0]) and orc.unary("relu6", x)[3] == 6
    assert np.array_equal(orc.cast(np.array([1.9, -1.9, nan, np.inf, 3e9], np.float32), "int32"),
                          np.array([1, -1, 0, 0, -1294967296], np.int32))
    # mean divides first, then sums (Mean.ts:37-48)
    v = np.array([[1e-45, 1e-45, 1e-45, 1e-45]], np.float32)
    assert orc.reduce("mean", v, 1)[0] == 0.0
    # matmul rounds once per 48-wide k-block (BatchMatMul.ts:108-119)
    a = np.ones((1, 96), np.float32)
    b = np.full((96, 1), np.float32(1 + 2 ** -20))
    exact = 96 * (1 + 2 ** -20)
    assert orc.batch_matmul(a, b)[0, 0] == np.float32(np.float32(48 * (1 + 2 ** -20)) * 2)
    assert abs(orc.batch_matmul(a, b)[0, 0] - exact) < 1e-4
    # avg pool divides by the number of in-bounds taps
    x = np.arange(9, dtype=np.float32).reshape(1, 3, 3, 1)
    assert orc.pool2d(x, "avg", 2, 1, "same")[0, 2, 2, 0] == 8.0
    with pytest.raises(ValueError):
        orc.gather(np.zeros((3, 2), np.float32), np.array([3], np.int32))


def test_float16_decoder_known_answers_and_every_bit_pattern():
    """io_utils_test.ts:601-616 and :711-778 (NaN, infinities, signed zeros, 0.25 / 0.5 /
    0.75 / 0.333), then all 65536 patterns against numpy's IEEE widening."""
    f = orc.decode_float16(np.array([13312, 14336, 14848], np.uint16))
    assert np.array_equal(f, np.float32([0.25, 0.5, 0.75]))
    assert np.isnan(orc.decode_float16(np.array([0x7e00], np.uint16))[0])
    inf = orc.decode_float16(np.array([0x7c00, 0xfc00], np.uint16))
    assert inf[0] == np.inf and inf[1] == -np.inf
    z = orc.decode_float16(np.array([0x0000, 0x8000], np.uint16))
    assert np.array_equal(z.view(np.uint32), np.array([0, 0x80000000], np.uint32))
    assert orc.decode_float16(np.array([0xfbff + 1], np.uint16))[0] == -np.inf
    assert orc.decode_float16(np.array([0x7bff + 1], np.uint16))[0] == np.inf
    v = orc.decode_float16(np.array([0x3400, 0x3800, 0x3a00, 0x3555], np.uint16))
    assert np.allclose(v, [0.25, 0.5, 0.75, 0.333], atol=5e-3)
    every = np.arange(65536, dtype=np.uint32).astype(np.uint16)
    got = orc.decode_float16(every)
    want = every.view(np.float16).astype(np.float32)
    nan = np.isnan(want)
    assert np.array_equal(np.isnan(got), nan)
    assert np.array_equal(got[~nan].view(np.uint32), want[~nan].view(np.uint32))
    # a NaN keeps its payload in the upper mantissa bits
    m = (every[nan].astype(np.uint32) & 0x3ff) << 13
    s = (every[nan].astype(np.uint32) & 0x8000) << 16
    assert np.array_equal(got[nan].view(np.uint32), s | 0x7f800000 | m)
