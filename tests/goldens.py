"""Loader for the committed golden fixtures (tests/golden/)."""
import json
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def _dec(v):
    if isinstance(v, dict) and set(v) == {"shape", "dtype", "data"}:
        conv = {"NaN": float("nan"), "Infinity": float("inf"), "-Infinity": float("-inf")}
        data = [conv[x] if isinstance(x, str) else x for x in v["data"]]
        return np.array(data, dtype=np.float64).astype(v["dtype"]).reshape(v["shape"])
    if isinstance(v, dict):
        return {k: _dec(x) for k, x in v.items()}
    if isinstance(v, list):
        return [_dec(x) for x in v]
    return v


def load_ts_goldens():
    with open(os.path.join(HERE, "golden", "ts_goldens.json")) as f:
        blob = json.load(f)
    return [_dec(c) for c in blob["cases"]], blob["summary"]


def case_id(c):
    return "%s:%d:%s" % (os.path.basename(c["file"]), c["line"], c["op"])


def arrays_close(actual, expected, eps):
    """tfjs-core/src/test_util.ts:139-147 (areClose) applied elementwise: two
    non-finite values always match; otherwise |a - e| <= eps and neither is NaN."""
    a = np.asarray(actual, np.float64).reshape(-1)
    e = np.asarray(expected, np.float64).reshape(-1)
    if a.size != e.size:
        return False, "size %d vs %d" % (a.size, e.size)
    both_nonfinite = ~np.isfinite(a) & ~np.isfinite(e)
    with np.errstate(invalid="ignore"):
        bad = ~both_nonfinite & (np.isnan(a) | np.isnan(e) | (np.abs(a - e) > eps))
    if bad.any():
        i = int(np.argmax(bad))
        return False, "index %d: actual %r expected %r" % (i, a[i], e[i])
    return True, ""
