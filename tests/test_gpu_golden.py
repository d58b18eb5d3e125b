"""The reference's own known-answer vectors, replayed through the CUDA backend.

fp32 math mode must meet the reference suite's absolute tolerance 1e-3
(tfjs-core/src/test_util.ts:23).  The default TF32 tensor-core mode is checked
with the same absolute bound plus the TF32 allowance 2e-3 * max|expected|.
"""
import numpy as np
import pytest

from tests import goldens, opcases

pytestmark = pytest.mark.gpu

CASES, _ = goldens.load_ts_goldens()


@pytest.mark.parametrize("case", CASES, ids=[goldens.case_id(c) for c in CASES])
def test_cuda_matches_reference_vector(cuda_engine, case):
    for mode in ("fp32", "tf32"):
        cuda_engine.backend.set_math_mode(mode)
        try:
            got = opcases.run_cuda(case)
        finally:
            cuda_engine.backend.set_math_mode("tf32")
        if case.get("squeeze0"):
            got = got[0]
        assert list(got.shape) == case["expected_shape"], mode
        finite = case["expected"][np.isfinite(case["expected"])]
        scale = float(np.max(np.abs(finite))) if finite.size else 0.0
        eps = 1e-3 if mode == "fp32" else 1e-3 + 2e-3 * scale
        ok, why = goldens.arrays_close(got, case["expected"], eps)
        assert ok, "%s: %s" % (mode, why)
