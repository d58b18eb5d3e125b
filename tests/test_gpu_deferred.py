"""Deferred launches of the CUDA backend (B200 only).

A FusedConv2D with a linear activation and a same-shape float32 Add are launched
when their result is first needed; an Add that consumes a pending convolution and a
Relu / Relu6 that consumes either fold into the producer's epilogue.  Each folded
form must give the bits of the separate kernels (every step rounds to fp32 in the
same order) and stay within the TF32 tolerance of the CPU oracle, and the
KernelBackend bookkeeping (data ids, reference counts) must look as if nothing had
been deferred.
"""
import ctypes
import zlib

import numpy as np
import pytest

from oracle import oracle as orc

pytestmark = pytest.mark.gpu

TF32_TOL = 2e-3


def _inputs(seed, xs, fs):
    r = np.random.default_rng(seed)
    fan_in = fs[0] * fs[1] * fs[2]
    x = r.standard_normal(xs).astype(np.float32)
    f = (r.standard_normal(fs) * np.sqrt(2.0 / fan_in)).astype(np.float32)
    b = (r.standard_normal(fs[3]) * 0.1).astype(np.float32)
    return x, f, b


def _block(tf, x, f, b, shortcut, strides, pad, post, conv_first=True, big=True):
    """conv(+bias, linear) -> Add(shortcut) -> post, through the op front ends."""
    xt = tf.tensor(x)
    ft = tf.tensor(f)
    bt = tf.tensor(b)
    st = tf.tensor(shortcut) if shortcut is not None else None
    y = tf.fused_conv2d(xt, ft, strides, pad, bias=bt, activation="linear")
    if st is not None:
        s = tf.add(y, st) if conv_first else tf.add(st, y)
        y.dispose()
        y = s
    if post is not None:
        z = getattr(tf, post)(y)
        y.dispose()
        y = z
    out = y.dataSync().reshape(y.shape)
    for t in (xt, ft, bt, st, y):
        if t is not None:
            t.dispose()
    return out


def _oracle_block(x, f, b, shortcut, strides, pad, post):
    ref = orc.fused_conv2d(x, f, strides, pad, bias=b, activation="linear")
    if shortcut is not None:
        ref = orc.binary("add", ref, shortcut)
    if post is not None:
        ref = orc.unary(post, ref)
    return ref


CASES = {
    # ResNet bottleneck exits: 1x1 expand, + identity shortcut, relu
    "pw_64_256_relu": ((4, 28, 28, 64), (1, 1, 64, 256), 1, "same", True, "relu"),
    "pw_512_2048_relu": ((2, 7, 7, 512), (1, 1, 512, 2048), 1, "same", True, "relu"),
    # MobileNetV2 linear bottleneck: projection, + shortcut, no activation
    "pw_144_24_linear": ((3, 28, 28, 144), (1, 1, 144, 24), 1, "same", True, None),
    "pw_relu6": ((2, 14, 14, 96), (1, 1, 96, 160), 1, "same", True, "relu6"),
    # basic block: 3x3 conv, + shortcut, relu; strided; ragged channel counts
    "c3_64_relu": ((2, 28, 28, 64), (3, 3, 64, 64), 1, "same", True, "relu"),
    "c3_s2_relu": ((2, 29, 29, 32), (3, 3, 32, 48), 2, "same", True, "relu"),
    "c3_tailN_relu": ((2, 13, 13, 24), (3, 3, 24, 36), 1, "valid", True, "relu"),
    "c3_oddN_relu": ((2, 9, 9, 8), (3, 3, 8, 13), 1, "same", True, "relu"),
    "stem_cin3_relu": ((2, 32, 32, 3), (3, 3, 3, 32), 2, "same", True, "relu"),
    # conv -> Relu with no Add in between
    "c3_relu_only": ((2, 28, 28, 64), (3, 3, 64, 64), 1, "same", False, "relu"),
    "pw_relu6_only": ((2, 14, 14, 96), (1, 1, 96, 160), 1, "same", False, "relu6"),
}


@pytest.mark.parametrize("name", sorted(CASES))
@pytest.mark.parametrize("conv_first", [True, False])
def test_folded_block_matches_separate_kernels_and_oracle(cuda_engine, name, conv_first):
    from tfjs_b200 import ops as tf
    xs, fs, strides, pad, with_add, post = CASES[name]
    if not with_add and not conv_first:
        pytest.skip("no Add in this case")
    x, f, b = _inputs(zlib.crc32(name.encode()) % 1000, xs, fs)
    backend = cuda_engine.backend
    ref_plain = orc.fused_conv2d(x, f, strides, pad, bias=b, activation="linear")
    shortcut = None
    if with_add:
        shortcut = np.random.default_rng(7).standard_normal(ref_plain.shape).astype(np.float32)
    assert backend.lazy_fusion
    before = backend.launch_count()
    folded = _block(tf, x, f, b, shortcut, strides, pad, post, conv_first)
    launches = backend.launch_count() - before
    backend.lazy_fusion = False
    try:
        before = backend.launch_count()
        eager = _block(tf, x, f, b, shortcut, strides, pad, post, conv_first)
        eager_launches = backend.launch_count() - before
    finally:
        backend.lazy_fusion = True
    assert np.array_equal(folded.view(np.uint32), eager.view(np.uint32))
    assert launches < eager_launches or (not with_add and post is None)
    ref = _oracle_block(x, f, b, shortcut, strides, pad, post)
    err = np.max(np.abs(folded.astype(np.float64) - ref)) / np.max(np.abs(ref))
    assert err <= TF32_TOL, err


def test_folded_block_fp32_math_mode(cuda_engine):
    """The SIMT fp32 GEMM carries the same epilogue."""
    from tfjs_b200 import ops as tf
    x, f, b = _inputs(3, (2, 14, 14, 32), (3, 3, 32, 40))
    ref_plain = orc.fused_conv2d(x, f, 1, "same", bias=b, activation="linear")
    shortcut = np.random.default_rng(8).standard_normal(ref_plain.shape).astype(np.float32)
    backend = cuda_engine.backend
    backend.set_math_mode("fp32")
    try:
        got = _block(tf, x, f, b, shortcut, 1, "same", "relu")
    finally:
        backend.set_math_mode("tf32")
    ref = _oracle_block(x, f, b, shortcut, 1, "same", "relu")
    assert np.max(np.abs(got - ref)) <= 2e-5 * np.max(np.abs(ref))


@pytest.mark.parametrize("post", [None, "relu", "relu6"])
@pytest.mark.parametrize("n", [1, 5, 4096, 1 << 20, (1 << 20) + 3])
def test_pending_add_is_bit_exact(cuda_engine, post, n):
    from tfjs_b200 import ops as tf
    r = np.random.default_rng(n)
    a = (r.standard_normal(n) * 4).astype(np.float32)
    b = (r.standard_normal(n) * 4).astype(np.float32)
    if n >= 5:
        a[:5] = [np.nan, -0.0, np.inf, -np.inf, 7.0]
        b[:5] = [1.0, 0.0, -np.inf, 1.0, -1.0]
    at, bt = tf.tensor(a), tf.tensor(b)
    y = tf.add(at, bt)
    if n * 4 > 4096:
        assert cuda_engine.backend.pending_of(y.dataId) is not None
    if post:
        z = getattr(tf, post)(y)
        y.dispose()
        y = z
    got = y.dataSync()
    ref = orc.binary("add", a, b)
    if post:
        ref = orc.unary(post, ref)
    ref = np.asarray(ref, np.float32)
    nan = np.isnan(ref)
    assert np.array_equal(np.isnan(got), nan)   # NaN payloads are not part of the contract
    assert np.array_equal(got[~nan].view(np.uint32), ref[~nan].view(np.uint32))
    for t in (at, bt, y):
        t.dispose()


def test_both_operands_pending_convolutions(cuda_engine):
    """Projection shortcut: both Add operands are pending convolutions."""
    from tfjs_b200 import ops as tf
    x, f1, b1 = _inputs(11, (2, 14, 14, 64), (1, 1, 64, 128))
    _, f2, b2 = _inputs(12, (2, 14, 14, 64), (1, 1, 64, 128))
    xt, f1t, b1t, f2t, b2t = [tf.tensor(v) for v in (x, f1, b1, f2, b2)]
    main = tf.fused_conv2d(xt, f1t, 1, "same", bias=b1t)
    proj = tf.fused_conv2d(xt, f2t, 1, "same", bias=b2t)
    s = tf.add(main, proj)
    y = tf.relu(s)
    for t in (main, proj, s, xt, f1t, b1t, f2t, b2t):
        t.dispose()
    got = y.dataSync().reshape(y.shape)
    y.dispose()
    ref = orc.unary("relu", orc.binary(
        "add", orc.fused_conv2d(x, f1, 1, "same", bias=b1, activation="linear"),
        orc.fused_conv2d(x, f2, 1, "same", bias=b2, activation="linear")))
    assert np.max(np.abs(got - ref)) <= TF32_TOL * np.max(np.abs(ref))


def test_pending_tensor_with_several_consumers(cuda_engine):
    """A pending result consumed by an Add, by a Relu and read back stays correct."""
    from tfjs_b200 import ops as tf
    x, f, b = _inputs(21, (2, 14, 14, 32), (3, 3, 32, 32))
    xt, ft, bt = tf.tensor(x), tf.tensor(f), tf.tensor(b)
    conv = tf.fused_conv2d(xt, ft, 1, "same", bias=bt)
    s = tf.add(conv, xt)          # folds the Add into a second pending convolution
    r = tf.relu(s)                # launches conv + add + relu
    r2 = tf.relu(conv)            # launches conv + relu
    m = tf.mul(s, s)              # launches conv + add, then the multiply
    plain = conv.dataSync().reshape(conv.shape)   # launches the convolution itself
    ref = orc.fused_conv2d(x, f, 1, "same", bias=b, activation="linear")
    tol = TF32_TOL * np.max(np.abs(ref))
    assert np.max(np.abs(plain - ref)) <= tol
    got_s = s.dataSync().reshape(s.shape)
    assert np.array_equal(got_s, plain + x)
    assert np.array_equal(r.dataSync().reshape(s.shape), np.maximum(got_s, 0))
    assert np.array_equal(r2.dataSync().reshape(s.shape), np.maximum(plain, 0))
    assert np.array_equal(m.dataSync().reshape(s.shape), got_s * got_s)
    for t in (conv, s, r, r2, m, xt, ft, bt):
        t.dispose()


def test_bookkeeping_hides_deferral(cuda_engine):
    """numDataBuffers / refCount as if the kernels had run eagerly; operands of a
    pending launch stay readable by it after the caller disposed them; disposing a
    never-launched result releases them."""
    from tfjs_b200 import ops as tf
    backend = cuda_engine.backend
    x, f, b = _inputs(31, (2, 14, 14, 32), (1, 1, 32, 64))
    base = cuda_engine.memory()
    xt, ft, bt = tf.tensor(x), tf.tensor(f), tf.tensor(b)
    y = tf.fused_conv2d(xt, ft, 1, "same", bias=bt)
    assert backend.pending_of(y.dataId) is not None
    assert backend.refCount(xt.dataId) == 1
    assert cuda_engine.memory()["numDataBuffers"] == base["numDataBuffers"] + 4
    xt.dispose(), ft.dispose(), bt.dispose()
    assert cuda_engine.memory()["numDataBuffers"] == base["numDataBuffers"] + 1
    assert cuda_engine.memory()["numTensors"] == base["numTensors"] + 1
    got = y.dataSync().reshape(y.shape)
    ref = orc.fused_conv2d(x, f, 1, "same", bias=b, activation="linear")
    assert np.max(np.abs(got - ref)) <= TF32_TOL * np.max(np.abs(ref))
    assert backend.pending_of(y.dataId) is None
    assert len(backend.data) == backend.numDataIds()
    y.dispose()
    after = cuda_engine.memory()
    assert after["numDataBuffers"] == base["numDataBuffers"]
    # never launched
    xt, ft, bt = tf.tensor(x), tf.tensor(f), tf.tensor(b)
    launches = backend.launch_count()
    y = tf.fused_conv2d(xt, ft, 1, "same", bias=bt)
    z = tf.add(y, y)
    for t in (xt, ft, bt, y, z):
        t.dispose()
    assert backend.launch_count() == launches
    assert len(backend.data) == backend.numDataIds() == base["numDataBuffers"]
    assert cuda_engine.memory()["numDeviceBuffers"] == base["numDeviceBuffers"]


def test_profile_names_folded_launches(cuda_engine):
    from tfjs_b200 import ops as tf
    x, f, b = _inputs(41, (2, 14, 14, 32), (1, 1, 32, 64))
    xt, ft, bt = tf.tensor(x), tf.tensor(f), tf.tensor(b)
    sc = tf.tensor(np.ones((2, 14, 14, 64), np.float32))

    def run():
        y = tf.fused_conv2d(xt, ft, 1, "same", bias=bt)
        s = tf.add(y, sc)
        r = tf.relu(s)
        y2 = tf.fused_conv2d(xt, ft, 1, "same", bias=bt)
        m = tf.mul(y2, sc)
        m.dataSync()                  # launches the convolution, then the multiply
        r.dataSync()                  # launches the convolution with the Add and the Relu
        for t in (y, s, y2):
            t.dispose()
        return r, m
    prof = cuda_engine.profile(run)
    names = [k["name"] for k in prof["kernels"] if not k["deferred"]]
    assert names == ["FusedConv2D", "Multiply", "FusedConv2D+Add+Relu"], names
    assert all(k["kernelTimeMs"] >= 0 for k in prof["kernels"])
    # the extra information of a record names the kernel instantiations it launched
    # (BackendTimingInfo.getExtraProfileInfo); deferred records launched nothing themselves
    launched = {k["name"]: k["extraInfo"] for k in prof["kernels"] if not k["deferred"]}
    assert "RES=1" in launched["FusedConv2D+Add+Relu"] and "gemm_tf32_kernel<" in launched["FusedConv2D"]
    assert "RES=0" in launched["FusedConv2D"]
    assert all(k["extraInfo"] == "" for k in prof["kernels"] if k["deferred"])
    for t in prof["result"] + (xt, ft, bt, sc):
        t.dispose()


def test_time_reports_kernel_ms_and_extra_profile_info(cuda_engine):
    """backend.time(f) is a BackendTimingInfo: kernelMs from CUDA events and
    getExtraProfileInfo() naming what ran."""
    from tfjs_b200 import ops as tf
    a = tf.tensor(np.ones((512, 512), np.float32))

    def work():
        b = tf.mat_mul(a, a)
        c = tf.softmax(b)
        c.dataSync()
        b.dispose()
        c.dispose()
    info = cuda_engine.backend.time(work)
    assert info["kernelMs"] > 0 and info["wallMs"] >= info["kernelMs"] * 0.5
    text = info["getExtraProfileInfo"]()
    assert "gemm_tf32_" in text and "softmax_kernel" in text
    # the log is off again: nothing accumulates outside time() / profile()
    tf.relu(a).dispose()
    assert cuda_engine.backend.launch_log_take() == ""
    a.dispose()


def test_residual_entry_point_rejects_bad_arguments(cuda_engine):
    from tfjs_b200 import _cabi
    backend = cuda_engine.backend
    lib = backend.lib
    x, f, b = _inputs(51, (1, 4, 4, 8), (1, 1, 8, 8))
    from tfjs_b200 import ops as tf
    xt, ft = tf.tensor(np.tile(x, (8, 1, 1, 1))), tf.tensor(np.tile(f, (1, 1, 1, 64)))
    out = backend.make_output([8, 4, 4, 512], "float32")
    small = backend.make_output([8, 4, 4, 8], "float32")
    p = _cabi.Conv2DParams()
    p.batch, p.in_h, p.in_w, p.in_c, p.out_h, p.out_w, p.out_c = 8, 4, 4, 8, 4, 4, 512
    p.filter_h = p.filter_w = p.stride_h = p.stride_w = p.dilation_h = p.dilation_w = 1
    p.activation = _cabi.ACTIVATIONS["linear"]
    ids = [backend.device_id(t.dataId) for t in (xt, ft)]
    o = backend.device_id(out.dataId)
    rc = lib.tfjs_cuda_fused_conv2d_residual(backend.ctx, ctypes.byref(p), ids[0], ids[1], 0, 0,
                                             0, _cabi.ACTIVATIONS["relu"], o)
    assert rc == 1
    rc = lib.tfjs_cuda_fused_conv2d_residual(backend.ctx, ctypes.byref(p), ids[0], ids[1], 0, 0,
                                             backend.device_id(small.dataId),
                                             _cabi.ACTIVATIONS["relu"], o)
    assert rc != _cabi.OK      # residual smaller than the output
    rc = lib.tfjs_cuda_fused_conv2d_residual(backend.ctx, ctypes.byref(p), ids[0], ids[1], 0, 0,
                                             o, _cabi.ACTIVATIONS["elu"], o)
    assert rc == 5
    rc = lib.tfjs_cuda_add_activation(backend.ctx, _cabi.ACTIVATIONS["sigmoid"], o, o,
                                      8 * 4 * 4 * 512, o)
    assert rc == 5
    backend.sync()
    for t in (xt, ft):
        t.dispose()
    backend.disposeData(out.dataId)
    backend.disposeData(small.dataId)


def test_async_read_overlaps_later_launches(cuda_engine):
    """tensor.data() returns at once; kernels launched afterwards do not disturb the
    bytes it delivers, tickets are collected once, and a small host-resident tensor
    resolves without touching the device."""
    from tfjs_b200 import ops as tf
    backend = cuda_engine.backend
    r = np.random.default_rng(61)
    a = r.standard_normal(1 << 20).astype(np.float32)
    at = tf.tensor(a)
    y = tf.mul(at, at)
    host = backend.pinned_empty([1 << 20], "float32")
    pending = y.data(into=host)
    z = tf.add(y, at)                 # launched while the copy is outstanding
    z2 = tf.relu(z)
    got = pending.wait()
    assert got is host or np.shares_memory(got, host)
    assert np.array_equal(got, a * a)
    assert np.array_equal(pending.wait(), a * a)      # a second wait is a no-op
    assert np.array_equal(z2.dataSync(), np.maximum(a * a + a, 0))
    small = tf.tensor(np.arange(4, dtype=np.float32))
    assert np.array_equal(small.data().wait(), np.arange(4, dtype=np.float32))
    rc = backend.lib.tfjs_cuda_read_wait(backend.ctx, 12345)
    assert rc == 1
    for t in (at, y, z, z2, small):
        t.dispose()


# ------------------------------------------------------ elementwise chains --
def _chain_cases():
    r = np.random.default_rng(5)
    R, C = 96, 772
    x = r.standard_normal((R, C)).astype(np.float32)
    mean = r.standard_normal((R, 1)).astype(np.float32)
    var = (r.random((R, 1)) + 0.1).astype(np.float32)
    gamma = r.standard_normal(C).astype(np.float32)
    beta = r.standard_normal(C).astype(np.float32)
    eps = np.float32(1e-12)

    def layer_norm_tail(tf, t):
        # the graph models' decomposed LayerNorm after the two Mean kernels
        inv = tf.rsqrt(tf.add(t["var"], t["eps"]))
        scale = tf.mul(inv, t["gamma"])
        return tf.add(tf.mul(t["x"], scale), tf.sub(t["beta"], tf.mul(t["mean"], scale)))

    def layer_norm_tail_simple(tf, t):
        # ((x - mean) * rstd) * gamma + beta, the form the converter leaves for tf.nn.moments
        norm = tf.mul(tf.sub(t["x"], t["mean"]), t["var"])
        return tf.add(tf.mul(norm, t["gamma"]), t["beta"])

    def gelu(tf, t):
        inner = tf.add(tf.erf(tf.mul(t["x"], t["c"])), t["one"])
        return tf.mul(tf.mul(t["x"], t["half"]), inner)

    def masked_scores(tf, t):
        return tf.add(tf.mul(t["s"], t["scale"]), t["mask"])

    def ragged(tf, t):        # sizes that are no multiples of 4: the scalar kernel
        return tf.relu(tf.sub(tf.square(t["p"]), tf.maximum(t["q"], t["row"])))

    def general_broadcast(tf, t):   # [3,1,5] op [1,4,1]: no addressing mode fits
        return tf.tanh(tf.add(tf.mul(t["u"], t["v"]), t["u"]))

    def long_chain(tf, t):    # more ops than one program holds
        y = t["x"]
        for i in range(40):
            y = tf.add(tf.mul(y, t["half"]), t["gamma"]) if i % 2 else tf.sub(y, t["beta"])
        return y

    def reused(tf, t):        # an intermediate with two consumers
        a = tf.exp(tf.mul(t["x"], t["half"]))
        return tf.div(tf.sub(a, t["one"]), tf.add(a, t["one"]))

    return {
        "layer_norm_tail": (layer_norm_tail, dict(x=x, mean=mean, var=var, gamma=gamma,
                                                  beta=beta, eps=eps)),
        "layer_norm_tail_simple": (layer_norm_tail_simple, dict(x=x, mean=mean, var=var,
                                                                gamma=gamma, beta=beta)),
        "gelu": (gelu, dict(x=x, c=np.float32(0.7071067811865476), one=np.float32(1),
                            half=np.float32(0.5))),
        "masked_scores": (masked_scores, dict(
            s=r.standard_normal((3, 4, 16, 32)).astype(np.float32), scale=np.float32(0.125),
            mask=r.standard_normal((3, 1, 1, 32)).astype(np.float32))),
        "ragged": (ragged, dict(p=r.standard_normal((7, 13)).astype(np.float32),
                                q=r.standard_normal((7, 13)).astype(np.float32),
                                row=r.standard_normal((7, 1)).astype(np.float32))),
        "general_broadcast": (general_broadcast, dict(
            u=r.standard_normal((3, 1, 5)).astype(np.float32),
            v=r.standard_normal((1, 4, 1)).astype(np.float32))),
        "long_chain": (long_chain, dict(x=x, half=np.float32(0.5), gamma=gamma, beta=beta)),
        "reused": (reused, dict(x=x, half=np.float32(0.5), one=np.float32(1))),
    }


class _OracleOps(object):
    """The op front ends evaluated by the CPU oracle on numpy arrays."""
    def __getattr__(self, name):
        binary = {"add": "add", "sub": "sub", "mul": "mul", "div": "div", "maximum": "maximum"}
        if name in binary:
            return lambda a, b: orc.binary(binary[name], a, b)
        return lambda a: orc.unary(name, a)


@pytest.mark.parametrize("name", sorted(_chain_cases()))
def test_elementwise_chain_matches_separate_kernels_and_oracle(cuda_engine, name):
    from tfjs_b200 import ops as tf
    fn, arrays = _chain_cases()[name]
    backend = cuda_engine.backend
    outs, launches = {}, {}
    for lazy in (True, False):
        backend.lazy_fusion = lazy
        try:
            tensors = {k: tf.tensor(v) for k, v in arrays.items()}
            before_t = cuda_engine.memory()["numTensors"]
            n0 = backend.launch_count()
            y = fn(tf, tensors)
            outs[lazy] = y.dataSync().reshape(y.shape)
            launches[lazy] = backend.launch_count() - n0
            y.dispose()
            for t in tensors.values():
                t.dispose()
        finally:
            backend.lazy_fusion = True
    assert np.array_equal(outs[True].view(np.uint32), outs[False].view(np.uint32)), name
    assert launches[True] <= launches[False]
    if name in ("layer_norm_tail", "layer_norm_tail_simple", "gelu", "masked_scores"):
        # chains the library has straight-line kernels for
        assert launches[True] < launches[False], (name, launches)
    ref = fn(_OracleOps(), arrays)
    ok = np.isfinite(ref)
    assert np.array_equal(np.isnan(outs[True]), np.isnan(ref))
    scale = max(float(np.max(np.abs(ref[ok]))), 1e-30)
    assert float(np.max(np.abs(outs[True][ok] - ref[ok]))) <= 1e-6 * scale, name


def test_fused_elementwise_rejects_malformed_programs(cuda_engine):
    from tfjs_b200 import _cabi
    backend = cuda_engine.backend
    out = backend.make_output([64], "float32")
    src = backend.make_output([64], "float32")
    prog = _cabi.EwProgram()
    prog.n_inputs, prog.n_ops, prog.n, prog.cols = 1, 1, 64, 64
    prog.input_id[0] = backend.device_id(src.dataId)
    prog.input_mode[0] = _cabi.EW_FULL
    prog.ops[0].opcode, prog.ops[0].a, prog.ops[0].b = 0, 0, 3        # operand slot 3 does not exist
    call = lambda: backend.lib.tfjs_cuda_fused_elementwise(
        backend.ctx, ctypes.byref(prog), backend.device_id(out.dataId))
    assert call() == 1
    prog.ops[0].b = 0
    prog.ops[0].opcode = 6                                            # Pow is not fusable
    assert call() == 1
    prog.ops[0].opcode = 0
    prog.input_mode[0], prog.input_period[0] = _cabi.EW_PERIODIC, 48   # 48 does not divide 64
    assert call() == 1
    prog.n_ops = 25
    assert call() == 1
    backend.disposeData(out.dataId)
    backend.disposeData(src.dataId)


def test_very_long_unread_chain_does_not_recurse_deeply(cuda_engine):
    """3000 dependent elementwise kernels with no read in between."""
    from tfjs_b200 import ops as tf
    x = tf.tensor(np.full(4096, 1.0, np.float32))
    one = tf.tensor(np.float32(1.0))
    y = x
    for _ in range(3000):
        z = tf.add(y, one)
        if y is not x:
            y.dispose()
        y = z
    assert np.array_equal(y.dataSync(), np.full(4096, 3001.0, np.float32))
    for t in (x, one, y):
        t.dispose()
