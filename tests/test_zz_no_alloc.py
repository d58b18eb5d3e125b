"""tfjs_cuda_dequantize_static: the dequantisation entry point for hosts that may
not allocate device memory (the lookup table is a fixed array inside the library).

Called straight through the C ABI, twice in a row with different quantised types
and parameters, and compared bit for bit with tfjs_cuda_dequantize on the same
inputs.  The second call would expose anything stale left in the shared table by
the first.  The file name sorts last so that a run that stops at the first failure
has already run every other test; the test also passes alone in a fresh process.
"""
from ctypes import byref, c_int32, c_uint64, c_void_p

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _upload(be, arr):
    out = c_int32()
    be.check(be.lib.tfjs_cuda_alloc(be.ctx, arr.nbytes, byref(out)))
    be.check(be.lib.tfjs_cuda_write(be.ctx, out.value, arr.ctypes.data_as(c_void_p), arr.nbytes))
    return out.value


def _pool_state(be):
    """(bytes handed out by the context, bytes the driver's pool has reserved, live buffers)."""
    v = [c_uint64() for _ in range(4)]
    be.check(be.lib.tfjs_cuda_memory(be.ctx, byref(v[0]), byref(v[1]), byref(v[2]), byref(v[3])))
    return v[0].value, v[1].value, v[3].value


def _run(be, fn, q, to_dtype, scale, mn, must_not_allocate=False):
    n = q.size
    q_id = _upload(be, q)
    out_id = c_int32()
    be.check(be.lib.tfjs_cuda_alloc(be.ctx, n * 4, byref(out_id)))
    before = _pool_state(be)
    be.check(fn(be.ctx, q.dtype.itemsize, to_dtype, q_id, scale, mn, n, out_id.value))
    if must_not_allocate:
        # neither the context's own accounting nor the driver pool's reservation moved
        # across the call (read before anything else touches the pool)
        assert _pool_state(be) == before
    host = np.empty(n, np.uint32)
    be.check(be.lib.tfjs_cuda_read(be.ctx, out_id.value, host.ctypes.data_as(c_void_p), n * 4))
    be.check(be.lib.tfjs_cuda_free(be.ctx, q_id))
    be.check(be.lib.tfjs_cuda_free(be.ctx, out_id.value))
    return host


def test_static_table_dequantize_matches_pool_version(cuda_engine):
    be = cuda_engine.backend
    lib = be.lib
    r = np.random.default_rng(99)
    n = 300007
    cases = [
        (r.integers(0, 65536, n).astype(np.uint16), 0, 3.1e-5, -1.0),   # float32 target
        (r.integers(0, 256, n).astype(np.uint8), 0, 0.0123, -1.57),     # narrower table next
        (r.integers(0, 256, n).astype(np.uint8), 1, 0.37, -40.25),      # int32 target
        (r.integers(0, 65536, n).astype(np.uint16), 1, 0.0417, -900.5),  # wide table, int32
    ]
    mem_before = c_uint64()
    be.check(lib.tfjs_cuda_memory(be.ctx, None, None, None, byref(mem_before)))
    for q, to_dtype, scale, mn in cases:
        # the static call goes first, so that in a fresh process the very first call on the
        # device (the one that looks up the table's address) is covered by the check too
        got = _run(be, lib.tfjs_cuda_dequantize_static, q, to_dtype, scale, mn,
                   must_not_allocate=True)
        want = _run(be, lib.tfjs_cuda_dequantize, q, to_dtype, scale, mn)
        assert np.array_equal(got, want)
    mem_after = c_uint64()
    be.check(lib.tfjs_cuda_memory(be.ctx, None, None, None, byref(mem_after)))
    assert mem_after.value == mem_before.value   # no tensor was left behind


def test_static_table_rejects_wider_types(cuda_engine):
    from tfjs_b200.backend import CudaError
    be = cuda_engine.backend
    q = np.zeros(64, np.uint8)
    q_id = _upload(be, q)
    out_id = c_int32()
    be.check(be.lib.tfjs_cuda_alloc(be.ctx, 64 * 4, byref(out_id)))
    with pytest.raises(CudaError, match="widest supported type is uint16"):
        be.check(be.lib.tfjs_cuda_dequantize_static(be.ctx, 4, 0, q_id, 1.0, 0.0, 16,
                                                    out_id.value))
    be.check(be.lib.tfjs_cuda_free(be.ctx, q_id))
    be.check(be.lib.tfjs_cuda_free(be.ctx, out_id.value))
