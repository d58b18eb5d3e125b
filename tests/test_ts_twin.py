"""The TypeScript package (tfjs_b200/ts) cannot be compiled or run here (no Node), so this
test holds it to the executed Python host layer and to the C header by reading its source:

  * the kernel names it registers are the names the Python layer registers;
  * its enum tables (activations, dtypes, unary / binary / reduce ops, weight storage,
    elementwise input modes) carry the header's values;
  * the byte offsets its DataView packers write are the offsets of the C structs as ctypes
    lays them out (conv2d params, matmul params, weight spec, elementwise program);
  * the N-API shim references every function the header declares, and every function the
    TypeScript side calls on the binding is exported by the shim;
  * the custom graph ops and the pending-launch classes exist under the same names.
"""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TS = os.path.join(ROOT, "tfjs_b200", "ts")


def _read(*parts):
    with open(os.path.join(TS, *parts)) as f:
        return f.read()


def _all_ts():
    out = {}
    for d, _, files in os.walk(os.path.join(TS, "src")):
        for f in files:
            if f.endswith(".ts"):
                out[os.path.relpath(os.path.join(d, f), TS)] = open(os.path.join(d, f)).read()
    return out


def _ts_table(src, name):
    m = re.search(r"export const %s\b[^=]*=\s*\{(.*?)\};" % name, src, re.S)
    assert m, name
    return {k: int(v) for k, v in re.findall(r"(\w+):\s*(-?\d+)", m.group(1))}


def test_kernel_names_match_the_python_layer():
    import tfjs_b200  # noqa: F401  (registers the kernels)
    from tfjs_b200 import kernel_registry
    py = set(c.kernelName for c in kernel_registry.get_kernels_for_backend("cuda"))
    src = "\n".join(_all_ts().values())
    ts = set(re.findall(r"kernelName:\s*'(\w+)'", src))
    # names given through tfjs-core's constants or a name list
    ts |= set(re.findall(r"config\((\w+),", src)) - {"kernelName"}
    ts |= set(re.findall(r"kernelName:\s*(_?[A-Z]\w+),", src))
    for lst in re.findall(r"(?:unaryNames|binaryNames)[^=]*=\s*\[(.*?)\];", src, re.S):
        ts |= set(re.findall(r"'(\w+)'", lst))
    assert ts == py, (sorted(py - ts), sorted(ts - py))


def test_enum_tables_match_the_header():
    from tfjs_b200 import _cabi
    src = _read("src", "binding.ts")
    act = _ts_table(src, "ACTIVATION")
    assert act == _cabi.ACTIVATIONS
    assert _ts_table(src, "DTYPE") == _cabi.DTYPES
    assert _ts_table(src, "BINARY_OP") == _cabi.BINARY_OPS
    assert _ts_table(src, "UNARY_OP") == _cabi.UNARY_OPS
    assert _ts_table(src, "REDUCE_OP") == _cabi.REDUCE_OPS
    assert _ts_table(src, "WEIGHT_STORAGE") == dict(raw=_cabi.STORED_RAW, uint8=_cabi.STORED_UINT8,
                                                    uint16=_cabi.STORED_UINT16,
                                                    float16=_cabi.STORED_FLOAT16)
    ew = _ts_table(src, "EW")
    assert ew == dict(FULL=_cabi.EW_FULL, PERIODIC=_cabi.EW_PERIODIC, ROW=_cabi.EW_ROW,
                      SCALAR=_cabi.EW_SCALAR, BATCHED=_cabi.EW_BATCHED,
                      MAX_INPUTS=_cabi.EW_MAX_INPUTS, MAX_OPS=_cabi.EW_MAX_OPS,
                      UNARY=_cabi.EW_UNARY)
    assert "STATUS_UNSUPPORTED = %d" % _cabi.UNSUPPORTED in src
    header = open(os.path.join(ROOT, "include", "tfjs_cuda.h")).read()
    for name, value in act.items():
        assert re.search(r"TFJS_CUDA_ACT_%s = %d\b" % (name.upper(), value), header), name


def _offsets(cls):
    return {n: getattr(cls, n).offset for n, _ in cls._fields_}


def test_struct_packers_write_the_c_layouts():
    from tfjs_b200 import _cabi
    src = _read("src", "binding.ts")
    conv = _offsets(_cabi.Conv2DParams)
    assert ctypes.sizeof(_cabi.Conv2DParams) == 80 and "new ArrayBuffer(80)" in src
    # 18 consecutive int32 fields from offset 0, then the double
    assert [conv[n] for n, _ in _cabi.Conv2DParams._fields_[:18]] == [4 * i for i in range(18)]
    assert "v.setFloat64(%d, leakyreluAlpha, true)" % conv["leakyrelu_alpha"] in src
    pend = _read("src", "pending.ts")
    assert "setInt32(%d, ACTIVATION[act], true)" % conv["activation"] in pend
    assert "setInt32(%d, biasLen, true)" % conv["bias_len"] in pend
    mm = _offsets(_cabi.MatMulParams)
    assert ctypes.sizeof(_cabi.MatMulParams) == 64 and "new ArrayBuffer(64)" in src
    assert [mm[n] for n, _ in _cabi.MatMulParams._fields_[:10]] == [4 * i for i in range(10)]
    for field, call in (("leakyrelu_alpha", "setFloat64(%d, leakyreluAlpha"),
                        ("gelu_scale", "setFloat32(%d, gelu[0]"), ("gelu_half", "setFloat32(%d, gelu[1]"),
                        ("gelu_one", "setFloat32(%d, gelu[2]"), ("gelu_divide", "setInt32(%d, gelu[3]")):
        assert call % mm[field] in src, field
    ws = _offsets(_cabi.WeightSpec)
    assert "new ArrayBuffer(%d * entries.length)" % ctypes.sizeof(_cabi.WeightSpec) in src
    for field, call in (("n", "setBigUint64(o,"), ("storage", "setInt32(o + %d, e.storage"),
                        ("dtype", "setInt32(o + %d, e.dtype"), ("scale", "setFloat64(o + %d, e.scale"),
                        ("min", "setFloat64(o + %d, e.min"), ("skip", "setInt32(o + %d, e.skip")):
        assert (call % ws[field] if "%d" in call else call) in src, field
    ew = _offsets(_cabi.EwProgram)
    assert "new ArrayBuffer(%d)" % ctypes.sizeof(_cabi.EwProgram) in src
    for field, call in (("n_inputs", "setInt32(%d, p.inputs.length"), ("n_ops", "setInt32(%d, p.ops.length"),
                        ("n", "setBigUint64(%d, BigInt(p.n)"), ("cols", "setUint32(%d, p.cols"),
                        ("input_id", "setInt32(%d + 4 * k, inp.id"),
                        ("input_mode", "setInt32(%d + 4 * k, inp.mode"),
                        ("input_period", "setUint32(%d + 4 * k, inp.period"),
                        ("input_aux", "setUint32(%d + 4 * k, inp.aux"),
                        ("ops", "const o = %d + 12 * j")):
        assert call % ew[field] in src, field
    assert ctypes.sizeof(_cabi.EwOp) == 12 and _offsets(_cabi.EwOp) == dict(opcode=0, a=2, b=3, p0=4, p1=8)
    assert "v.setInt16(o, op.opcode, true)" in src and "v.setUint8(o + 2, op.a)" in src


def test_shim_covers_the_header_and_the_typescript_calls():
    header = open(os.path.join(ROOT, "include", "tfjs_cuda.h")).read()
    declared = set(re.findall(r"^(?:int|void|const char\*)\s+(tfjs_cuda_\w+)\(", header, re.M))
    shim = _read("binding", "tfjs_cuda_binding.cc")
    used = set(re.findall(r"\b(tfjs_cuda_\w+)\(", shim))
    assert declared - used == set(), sorted(declared - used)
    exported = set(re.findall(r'\{"(\w+)",\s*\w+\}', shim))
    interface = set(re.findall(r"^  (\w+)\(", re.search(r"export interface CudaBinding \{(.*?)^\}",
                                                         _read("src", "binding.ts"), re.S | re.M).group(1), re.M))
    assert interface == exported, (sorted(interface - exported), sorted(exported - interface))
    called = set()
    for src in _all_ts().values():
        called |= set(re.findall(r"\bbinding\.(\w+)\b", src))
    assert called - exported == set(), sorted(called - exported)


def test_graph_ops_and_pending_classes_have_their_python_twins():
    from tfjs_b200 import backend, graph_model
    ts = _all_ts()
    pend = ts["src/pending.ts"]
    for cls in ("PendingConv", "PendingDepthwise", "PendingMatMul", "PendingTile", "PendingEw"):
        assert hasattr(backend, cls) and "export class %s" % cls in pend
    assert "export function canonicalProgram" in pend and hasattr(backend, "_canonical_program")
    rewrites = ts["src/graph_rewrites.ts"]
    for py, tsname in (("fuse_layer_norms", "fuseLayerNorms"), ("fuse_attention_heads", "fuseAttentionHeads"),
                       ("fuse_softmax_inputs", "fuseSoftmaxInputs"),
                       ("fuse_attention", "fuseAttention"),
                       ("fuse_gelu_into_matmul", "fuseGeluIntoMatMul"),
                       ("hoist_shared_operand_matmuls", "hoistSharedOperandMatMuls")):
        assert hasattr(graph_model, py) and "export function %s" % tsname in rewrites
    for op in ("_FusedLayerNorm", "_MatMulHeads", "_SoftmaxScaledMasked", "_FusedAttention",
               "_FusedMatMulGelu"):
        assert "registerOp('%s'" % op in rewrites
        assert 'op == "%s"' % op in open(os.path.join(ROOT, "tfjs_b200", "graph_model.py")).read()
    replay = ts["src/graph_model_cuda.ts"]
    for call in ("captureBegin", "captureEnd", "graphLaunch", "graphDestroy", "highWaterReset"):
        assert "binding.%s(" % call in replay
    io_ts = ts["src/io_cuda.ts"]
    for call in ("weightsBegin", "weightsPush", "weightsPushFile", "weightsEnd"):
        assert "binding.%s(" % call in io_ts
