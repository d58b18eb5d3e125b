"""The C-ABI library builds, loads, and exports every symbol the header declares."""
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "tfjs_cuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tfjs_cuda_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported_and_bound():
    from tfjs_b200 import _cabi
    lib = _cabi.load()
    declared = _declared_symbols()
    assert len(declared) >= 30
    for name in declared:
        assert hasattr(lib, name), "libtfjs_cuda.so does not export %s" % name
        assert name in _cabi.SIGNATURES, "no ctypes signature for %s" % name
    assert sorted(_cabi.SIGNATURES) == declared


def test_no_gpu_is_reported_not_faked():
    """Without a GPU, creating a backend raises; nothing falls back to the CPU."""
    import ctypes
    from tfjs_b200 import _cabi
    from tfjs_b200.backend import CudaBackend, CudaError
    lib = _cabi.load()
    n = ctypes.c_int(-1)
    lib.tfjs_cuda_device_count(ctypes.byref(n))
    if n.value == 0:
        try:
            CudaBackend(0)
        except CudaError:
            return
        raise AssertionError("CudaBackend(0) must fail when no GPU is present")


def test_product_does_not_import_oracle():
    pkg = os.path.join(ROOT, "tfjs_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                src = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in src.lower(), "%s mentions the oracle" % f
