"""`backend.read` of a large tensor (tfjs_cuda_read_begin / read_wait: the promise of
tfjs-core/src/backends/backend.ts:104) leaves the device through a staging copy on a stream
of its own, so the kernels launched behind it run while the bytes travel.  The tensor may be
disposed, and its memory rewritten, as soon as the call has returned."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n", [3 << 20, 1 << 18])     # 12 MB: staged; 1 MB: on the compute stream
def test_download_survives_dispose_and_reuse_of_the_block(cuda_engine, n):
    from tfjs_b200 import ops as tf
    be = cuda_engine.backend
    x = np.arange(n, dtype=np.float32)
    t, two, three = tf.tensor(x), tf.tensor(np.float32(2)), tf.tensor(np.float32(3))
    before = be.numDataIds()
    y = tf.mul(t, two)
    host = be.pinned_empty(y.shape, "float32")
    host[...] = -1
    pending = y.data(into=host)
    y.dispose()
    # blocks of the same size are handed out again at once and rewritten
    others = [tf.mul(t, three) for _ in range(4)]
    vals = [o.dataSync() for o in others]
    pending.wait()
    assert np.array_equal(host, x * 2)
    for v in vals:
        assert np.array_equal(v, x * 3)
    for o in others:
        o.dispose()
    assert be.numDataIds() == before
    for s in (t, two, three):
        s.dispose()


def test_sync_covers_a_staged_download(cuda_engine):
    from tfjs_b200 import ops as tf
    be = cuda_engine.backend
    x = np.random.default_rng(0).standard_normal(2 << 20).astype(np.float32)
    t = tf.tensor(x)
    y = tf.relu(t)
    host = be.pinned_empty(y.shape, "float32")
    pending = y.data(into=host)
    be.sync()                                   # not the ticket's wait
    assert np.array_equal(host, np.maximum(x, 0))
    pending.wait()
    for s in (t, y):
        s.dispose()
