"""Extracts known-answer vectors from the reference's own op tests.

Run in the container that has the reference checkout:

    python tests/golden/make_ts_goldens.py <tfjs checkout> tests/golden/ts_goldens.json

The reference's op tests (tfjs-core/src/ops/**/*_test.ts) hold inputs and
expected outputs inline.  Node is not available, so this script translates each
jasmine spec body from TypeScript into Python with a small rule-based
translator and executes it against a recording stand-in for the `tf` namespace.
Every `expectArraysClose(await t.data(), expected)` whose tensor `t` came out
of an op on the inference hot path becomes one golden case

    {file, line, spec, op, inputs, attrs, expected, expected_shape}

with `expected` taken verbatim from the reference test.  Specs that use things
outside the hot path (gradients, NCHW, complex, strings, browser pixels) or
that the translator cannot handle are skipped and counted in the summary that
is stored next to the cases.  The stand-in evaluates ops with the CPU oracle
only to feed later ops of the same spec; the expected values never come from it.
"""
import json
import math
import os
import re
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from tests import opcases  # noqa: E402

TEST_FILES = [
    "tfjs-core/src/ops/fused/fused_conv2d_test.ts",
    "tfjs-core/src/ops/fused/fused_mat_mul_test.ts",
    "tfjs-core/src/ops/fused/fused_depthwise_conv2d_test.ts",
    "tfjs-core/src/ops/mat_mul_test.ts",
    "tfjs-core/src/ops/conv2d_test.ts",
    "tfjs-core/src/ops/depthwise_conv2d_test.ts",
    "tfjs-core/src/ops/max_pool_test.ts",
    "tfjs-core/src/ops/avg_pool_test.ts",
    "tfjs-core/src/ops/softmax_test.ts",
    "tfjs-core/src/ops/gather_test.ts",
    "tfjs-core/src/ops/arg_max_test.ts",
    "tfjs-core/src/ops/mean_test.ts",
    "tfjs-core/src/ops/sum_test.ts",
    "tfjs-core/src/ops/max_test.ts",
    "tfjs-core/src/ops/add_test.ts",
    "tfjs-core/src/ops/relu_test.ts",
    "tfjs-core/src/ops/relu6_test.ts",
    "tfjs-core/src/ops/elu_test.ts",
    "tfjs-core/src/ops/sigmoid_test.ts",
    "tfjs-core/src/ops/leaky_relu_test.ts",
    "tfjs-core/src/ops/erf_test.ts",
    "tfjs-core/src/ops/exp_test.ts",
    "tfjs-core/src/ops/sqrt_test.ts",
    "tfjs-core/src/ops/rsqrt_test.ts",
    "tfjs-core/src/ops/square_test.ts",
    "tfjs-core/src/ops/tanh_test.ts",
    "tfjs-core/src/ops/transpose_test.ts",
    "tfjs-core/src/ops/batchnorm_test.ts",
    "tfjs-core/src/ops/clip_by_value_test.ts",
    "tfjs-core/src/ops/tile_test.ts",
    "tfjs-core/src/ops/binary_ops_test.ts",
    "tfjs-core/src/ops/arithmetic_test.ts",
    "tfjs-core/src/ops/sub_test.ts",
    "tfjs-core/src/ops/neg_test.ts",
    "tfjs-core/src/ops/abs_test.ts",
    "tfjs-core/src/ops/log_test.ts",
    "tfjs-core/src/ops/concat_test.ts",
    "tfjs-core/src/ops/slice_test.ts",
    "tfjs-core/src/ops/slice1d_test.ts",
    "tfjs-core/src/ops/slice2d_test.ts",
    "tfjs-core/src/ops/slice3d_test.ts",
    "tfjs-core/src/ops/slice4d_test.ts",
    "tfjs-core/src/ops/pad_test.ts",
    "tfjs-core/src/ops/stack_test.ts",
    "tfjs-core/src/ops/expand_dims_test.ts",
    "tfjs-core/src/tensor_test.ts",
]


class Skip(Exception):
    pass


# --------------------------------------------------------------- translator --
def strip_comments(src):
    out, i, n = [], 0, len(src)
    while i < n:
        c = src[i]
        if c in "'\"`":
            j = i + 1
            while j < n and src[j] != c:
                j += 2 if src[j] == "\\" else 1
            out.append(src[i:j + 1])
            i = j + 1
        elif src.startswith("//", i):
            while i < n and src[i] != "\n":
                i += 1
        elif src.startswith("/*", i):
            i = src.index("*/", i) + 2
        else:
            out.append(c)
            i += 1
    return "".join(out)


def match_close(src, i):
    """Index of the bracket closing the one at src[i]."""
    pairs = {"(": ")", "[": "]", "{": "}"}
    stack = []
    n = len(src)
    while i < n:
        c = src[i]
        if c in "'\"`":
            j = i + 1
            while src[j] != c:
                j += 2 if src[j] == "\\" else 1
            i = j
        elif c in pairs:
            stack.append(pairs[c])
        elif c in ")]}":
            if not stack or stack.pop() != c:
                raise Skip("unbalanced brackets")
            if not stack:
                return i
        i += 1
    raise Skip("unbalanced brackets")


def split_top(src, sep):
    """Split at `sep` characters that are outside brackets and strings."""
    parts, depth, start, i, n = [], 0, 0, 0, len(src)
    while i < n:
        c = src[i]
        if c in "'\"`":
            j = i + 1
            while src[j] != c:
                j += 2 if src[j] == "\\" else 1
            i = j
        elif c in "([{":
            depth += 1
        elif c in ")]}":
            depth -= 1
        elif c == sep and depth == 0:
            parts.append(src[start:i])
            start = i + 1
        i += 1
    parts.append(src[start:])
    return parts


def find_specs(src):
    """Yields (name, line, body) for every `it(...)` with an arrow-function body."""
    for m in re.finditer(r"(?m)^\s*it\(", src):
        start = m.end() - 1
        try:
            end = match_close(src, start)
        except Skip:
            continue
        inner = src[start + 1:end]
        arrow = inner.find("=>")
        if arrow < 0:
            continue
        name_part = inner[:arrow]
        head = name_part.rsplit("async", 1)[0]
        names = re.findall("'([^']*)'|\"([^\"]*)\"", head)
        name = "".join(a or b for a, b in names) or "?"
        brace = inner.find("{", arrow)
        if brace < 0:
            continue
        close = match_close(inner, brace)
        yield name.strip(), src.count("\n", 0, m.start()) + 1, inner[brace + 1:close], m.start()


def find_setups(src):
    """(span start, span end, body) of every `beforeEach(() => {...})`, the span being the
    describe block that holds it: its statements run before each spec of that block."""
    spans = []
    for m in re.finditer(r"\b(?:describeWithFlags|describe)\(", src):
        try:
            spans.append((m.start(), match_close(src, m.end() - 1)))
        except Skip:
            continue
    out = []
    for m in re.finditer(r"\bbeforeEach\(", src):
        try:
            end = match_close(src, m.end() - 1)
            inner = src[m.end():end]
            arrow = inner.find("=>")
            brace = inner.find("{", arrow)
            if arrow < 0 or brace < 0:
                continue
            body = inner[brace + 1:match_close(inner, brace)]
        except Skip:
            continue
        holders = [sp for sp in spans if sp[0] < m.start() < sp[1]]
        if holders:
            a, b = max(holders, key=lambda sp: sp[0])     # innermost
            out.append((a, b, body))
    return out


def strip_as_casts(e):
    out, i = [], 0
    while True:
        m = re.search(r"\s+as\s+", e[i:])
        if not m:
            out.append(e[i:])
            break
        out.append(e[i:i + m.start()])
        j = i + m.end()
        # skip one type expression
        if e[j] == "[":
            j = match_close(e, j) + 1
        else:
            mm = re.match(r"[A-Za-z_][\w.]*", e[j:])
            j += mm.end() if mm else 0
            if j < len(e) and e[j] == "<":
                depth = 0
                while True:
                    depth += e[j] == "<"
                    depth -= e[j] == ">"
                    j += 1
                    if depth == 0:
                        break
        while e.startswith("[]", j):
            j += 2
        i = j
    return "".join(out)


def convert_objects(e):
    """{a, b: c} -> dict(a=a, b=c), recursively."""
    out, i = [], 0
    while i < len(e):
        c = e[i]
        if c in "'\"`":
            j = i + 1
            while e[j] != c:
                j += 2 if e[j] == "\\" else 1
            out.append(e[i:j + 1])
            i = j + 1
        elif c == "{":
            j = match_close(e, i)
            items = []
            for part in split_top(e[i + 1:j], ","):
                part = part.strip()
                if not part:
                    continue
                kv = split_top(part, ":")
                if len(kv) == 1:
                    if not re.match(r"^[A-Za-z_]\w*$", part):
                        raise Skip("object literal")
                    items.append("%s=%s" % (part, part))
                else:
                    key = kv[0].strip().strip("'\"")
                    items.append("%s=%s" % (key, convert_objects(":".join(kv[1:]).strip())))
            out.append("dict(%s)" % ", ".join(items))
            i = j + 1
        else:
            out.append(c)
            i += 1
    return "".join(out)


def convert_ternary(e):
    parts = split_top(e, "?")
    if len(parts) == 1:
        return e
    if len(parts) != 2:
        raise Skip("nested ternary")
    ab = split_top(parts[1], ":")
    if len(ab) != 2:
        raise Skip("ternary")
    return "(%s if %s else %s)" % (ab[0].strip(), parts[0].strip(), ab[1].strip())


def tr_expr(e):
    e = e.strip()
    if "=>" in e or "function" in e:
        raise Skip("closure")
    e = strip_as_casts(e)
    e = re.sub(r"\bawait\s+", "", e)
    e = re.sub(r"\bnew\s+(Float32Array|Int32Array|Uint8Array)\s*\(", "__typed(", e)
    e = re.sub(r"\bnew\s+Array\s*\(", "__newarray(", e)
    e = re.sub(r"\bArray\.from\(", "__arrayfrom(", e)
    e = e.replace("tf.test_util.", "")
    e = e.replace("===", "==").replace("!==", "!=")
    e = re.sub(r"&&", " and ", e)
    e = re.sub(r"\|\|", " or ", e)
    e = re.sub(r"(?<![\w.])!(?!=)", " not ", e)
    e = re.sub(r"\bNaN\b", "__nan", e)
    e = re.sub(r"(?<![\w.])-?Infinity\b", lambda m: "(-__inf)" if m.group(0)[0] == "-" else "__inf", e)
    e = re.sub(r"\bNumber\.(POSITIVE|NEGATIVE)_INFINITY\b",
               lambda m: "__inf" if m.group(1) == "POSITIVE" else "(-__inf)", e)
    e = re.sub(r"\btrue\b", "True", e)
    e = re.sub(r"\bfalse\b", "False", e)
    e = re.sub(r"\b(null|undefined)\b", "None", e)
    e = re.sub(r"\bMath\.", "__math.", e)
    e = re.sub(r"([A-Za-z_][\w.]*)\.length\b", r"len(\1)", e)
    e = re.sub(r"\.push\(", ".append(", e)
    e = re.sub(r"<[A-Za-z_][\w.]*(\.[A-Za-z_]\w*)*>\(", "(", e)  # generic call args
    e = convert_objects(e)
    e = convert_ternary(e)
    return e


def split_statements(body):
    """Top-level statements of a block; `for` loops keep their block."""
    stmts, i, n = [], 0, len(body)
    while i < n:
        while i < n and body[i] in " \t\r\n;":
            i += 1
        if i >= n:
            break
        m = re.match(r"(for|if|while)\s*\(", body[i:])
        if m:
            p = i + m.end() - 1
            q = match_close(body, p)
            k = q + 1
            while body[k] in " \t\r\n":
                k += 1
            if body[k] != "{":
                raise Skip("unbraced block")
            r = match_close(body, k)
            stmts.append((m.group(1), body[p + 1:q], body[k + 1:r]))
            i = r + 1
            if m.group(1) == "if":
                mm = re.match(r"\s*else\b", body[i:])
                if mm:
                    raise Skip("else")
            continue
        # plain statement up to ';' at depth 0
        depth, j = 0, i
        while j < n:
            c = body[j]
            if c in "'\"`":
                k = j + 1
                while body[k] != c:
                    k += 2 if body[k] == "\\" else 1
                j = k
            elif c in "([{":
                depth += 1
            elif c in ")]}":
                depth -= 1
            elif c == ";" and depth == 0:
                break
            j += 1
        stmts.append(("stmt", body[i:j], None))
        i = j + 1
    return stmts


def tr_stmt(s):
    s = " ".join(s.split())
    m = re.match(r"^(const|let|var)\s+(.*)$", s)
    if m:
        s = m.group(2)
        # destructuring or typed declaration
        eq = None
        depth = 0
        for idx, c in enumerate(s):
            if c in "([{<":
                depth += 1
            elif c in ")]}>":
                depth -= 1
            elif c == "=" and depth == 0 and s[idx + 1] != "=" and s[idx - 1] not in "=!<>":
                eq = idx
                break
        if eq is None:
            name = re.match(r"[A-Za-z_]\w*", s).group(0)
            return "%s = None" % name
        lhs, rhs = s[:eq].strip(), s[eq + 1:].strip()
        if lhs.startswith("{") or lhs.startswith("["):
            if lhs.startswith("{"):
                names = [p.strip() for p in lhs.strip("{} ").split(",") if p.strip()]
                tmp = "__d"
                return "%s = %s\n%s" % (tmp, tr_expr(rhs), "\n".join(
                    "%s = %s['%s']" % (nm, tmp, nm) for nm in names))
            return "%s = %s" % (lhs, tr_expr(rhs))
        name = re.match(r"[A-Za-z_]\w*", lhs).group(0)
        return "%s = %s" % (name, tr_expr(rhs))
    m = re.match(r"^return\b\s*(.*)$", s)
    if m:
        e = tr_expr(m.group(1)) if m.group(1) else "None"
        return "return __obj(%s)" % e if e.startswith("dict(") else "return %s" % e
    m = re.match(r"^expect\((.*)\)\.toEqual\((.*)\)$", s)
    if m:
        return "__expect_equal(%s, %s)" % (tr_expr(m.group(1)), tr_expr(m.group(2)))
    m = re.match(r"^expect\((.*)\)\.toBe\((.*)\)$", s)
    if m:
        return "__expect_equal(%s, %s)" % (tr_expr(m.group(1)), tr_expr(m.group(2)))
    if s.startswith("expect("):
        raise Skip("expect form")
    m = re.match(r"^(\w+)\[([^\]]+)\]\s*=(?!=)\s*(.*)$", s)
    if m and not s.startswith("expectArrays"):
        # a JavaScript array grows when an index beyond its end is assigned
        return "__setidx(%s, %s, %s)" % (m.group(1), tr_expr(m.group(2)), tr_expr(m.group(3)))
    m = re.match(r"^(\w[\w.\[\]]*)\s*(\+|-|\*)?=\s*(.*)$", s)
    if m and not s.startswith("expectArrays"):
        return "%s %s= %s" % (tr_expr(m.group(1)), m.group(2) or "", tr_expr(m.group(3)))
    m = re.match(r"^(\w+)(\+\+|--)$", s)
    if m:
        return "%s %s= 1" % (m.group(1), m.group(2)[0])
    return tr_expr(s)


def tr_block(body, indent=0):
    lines = []
    pad = "    " * indent
    for kind, a, b in split_statements(body):
        if kind == "stmt":
            for ln in tr_stmt(a).split("\n"):
                lines.append(pad + ln)
        elif kind == "for":
            parts = split_top(a, ";")
            if len(parts) != 3:
                raise Skip("for form")
            m = re.match(r"^\s*(?:let|var|const)\s+(\w+)\s*=\s*(.*)$", parts[0].strip())
            c = re.match(r"^\s*(\w+)\s*(<=|<)\s*(.*)$", parts[1].strip())
            inc = parts[2].strip()
            if not m or not c or c.group(1) != m.group(1):
                raise Skip("for form")
            step = "1"
            if re.match(r"^(\+\+%s|%s\+\+)$" % (m.group(1), m.group(1)), inc):
                step = "1"
            else:
                mm = re.match(r"^%s\s*\+=\s*(.*)$" % m.group(1), inc)
                if not mm:
                    raise Skip("for increment")
                step = tr_expr(mm.group(1))
            hi = tr_expr(c.group(3)) + (" + 1" if c.group(2) == "<=" else "")
            lines.append("%sfor %s in range(int(%s), int(%s), int(%s)):" %
                         (pad, m.group(1), tr_expr(m.group(2)), hi, step))
            inner = tr_block(b, indent + 1)
            lines.extend(inner if inner else [pad + "    pass"])
        elif kind == "if":
            lines.append("%sif %s:" % (pad, tr_expr(a)))
            inner = tr_block(b, indent + 1)
            lines.extend(inner if inner else [pad + "    pass"])
        else:
            raise Skip("while")
    return lines


# ------------------------------------------------------- recording tf stand-in --
class FT(object):
    """Tensor stand-in: value, dtype, and the op case that produced it."""

    def __init__(self, value, dtype, case=None):
        self.value = value
        self.dtype = dtype
        self.case = case

    @property
    def shape(self):
        return list(self.value.shape)

    @property
    def rank(self):
        return self.value.ndim

    @property
    def size(self):
        return int(self.value.size)

    def data(self):
        return Data(self)

    def dataSync(self):
        return Data(self)

    def array(self):
        return self.value.tolist()

    def arraySync(self):
        return self.value.tolist()

    def buffer(self):
        return Buf(self.value)

    def bufferSync(self):
        return Buf(self.value)

    def reshape(self, shape):
        # a view of an op result still checks that op: the expected values are compared
        # flat, and the case keeps the op's own output shape
        out = FT(self.value.reshape(shape), self.dtype, self.case)
        out.op_shape = getattr(self, "op_shape", list(self.value.shape))
        if getattr(self, "squeeze0", False):
            out.squeeze0 = True
        return out

    def as1D(self):
        return self.reshape([-1])

    def as2D(self, a, b):
        return self.reshape([a, b])

    def as3D(self, a, b, c):
        return self.reshape([a, b, c])

    def as4D(self, a, b, c, d):
        return self.reshape([a, b, c, d])

    def flatten(self):
        return self.reshape([-1])

    def dispose(self):
        pass

    def clone(self):
        return FT(self.value.copy(), self.dtype, None)

    def toInt(self):
        return self.tf.cast(self, "int32")

    def toFloat(self):
        return self.tf.cast(self, "float32")

    def toBool(self):
        return self.tf.cast(self, "bool")

    def asType(self, dtype):
        return self.tf.cast(self, dtype)

    def __getattr__(self, name):
        # chained form a.op(b, ...) of tf.op(a, b, ...)
        if name.startswith("__") or name in ("tf", "squeeze0", "op_shape"):
            raise AttributeError(name)
        fn = getattr(self.tf, name, None)
        if fn is None:
            raise Skip("chained %s" % name)
        return lambda *args, **kw: fn(self, *args, **kw)


class Buf(object):
    """TensorBuffer stand-in (tfjs-core/src/tensor.ts TensorBuffer.get)."""

    def __init__(self, value):
        self.value = value

    def get(self, *idx):
        return float(self.value[tuple(int(i) for i in idx)]) if idx else float(self.value)


class Data(object):
    def __init__(self, t):
        self.t = t


def flat(v):
    if isinstance(v, Data):
        raise Skip("data as values")
    if isinstance(v, FT):
        raise Skip("tensor as values")
    return np.asarray(v)


def mk(values, shape=None, dtype=None):
    if isinstance(values, FT):
        raise Skip("tensor from tensor")
    arr = np.asarray(values)
    if arr.dtype == object:
        raise Skip("ragged values")
    if dtype in (None,):
        if arr.dtype == np.bool_:
            dtype = "bool"
        else:
            dtype = "float32"
    if dtype not in ("float32", "int32", "bool"):
        raise Skip("dtype %s" % dtype)
    npdt = {"float32": np.float32, "int32": np.int32, "bool": np.bool_}[dtype]
    if dtype == "int32":
        arr = np.trunc(np.nan_to_num(arr.astype(np.float64), nan=0.0, posinf=0.0, neginf=0.0))
    arr = arr.astype(npdt)
    if shape is not None:
        arr = arr.reshape([int(s) for s in shape])
    return FT(np.ascontiguousarray(arr), dtype)


def as_ft(v, dtype=None):
    if isinstance(v, FT):
        return v
    if isinstance(v, Data):
        raise Skip("data as tensor")
    return mk(v, None, dtype)


class Recorder(object):
    def __init__(self):
        self.cases = []

    def op(self, name, inputs, attrs, out_dtype="float32"):
        case = {"op": name, "inputs": {}, "attrs": attrs}
        dtypes = {}
        for k, v in inputs.items():
            if v is None:
                continue
            if isinstance(v, list):
                case["inputs"][k] = [t.value for t in v]
                dtypes[k] = [t.dtype for t in v]
            else:
                case["inputs"][k] = v.value
                dtypes[k] = v.dtype
        try:
            val = opcases.run_oracle(case)
        except NotImplementedError as e:
            raise Skip("not on the hot path: %s" % e)
        except Exception as e:
            raise Skip("op raised: %s" % str(e)[:60])
        case["input_dtypes"] = dtypes
        return FT(np.asarray(val), out_dtype, case)


def make_tf(rec):
    class NS(object):
        pass
    tf = NS()

    def tensor_n(n):
        def f(values, shape=None, dtype=None):
            if isinstance(shape, str):
                shape, dtype = None, shape
            t = mk(values, shape, dtype)
            if n is not None and t.value.ndim != n:
                if shape is None and n == 1:
                    t = FT(t.value.reshape(-1), t.dtype)
                elif t.value.ndim != n:
                    raise Skip("rank mismatch")
            return t
        return f
    for n in range(1, 7):
        setattr(tf, "tensor%dd" % n, tensor_n(n))
    tf.tensor = tensor_n(None)
    tf.scalar = lambda v, dtype=None: mk(v, [], dtype)
    tf.zeros = lambda shape, dtype="float32": mk(np.zeros(shape), shape, dtype)
    tf.ones = lambda shape, dtype="float32": mk(np.ones(shape), shape, dtype)
    tf.fill = lambda shape, v, dtype="float32": mk(np.full(shape, v), shape, dtype)
    tf.range = lambda a, b, step=1, dtype="float32": mk(np.arange(a, b, step), None, dtype)

    def fused_conv(opname):
        def f(d):
            if d.get("dataFormat", "NHWC") not in (None, "NHWC"):
                raise Skip("NCHW")
            x = as_ft(d["x"])
            attrs = {"strides": d.get("strides"), "pad": d.get("pad"),
                     "dilations": d.get("dilations") or [1, 1],
                     "dimRoundingMode": d.get("dimRoundingMode"),
                     "activation": d.get("activation") or "linear",
                     "leakyreluAlpha": d.get("leakyreluAlpha")}
            x3 = x.rank == 3
            xx = FT(x.value[None], x.dtype) if x3 else x
            out = rec.op(opname, {"x": xx, "filter": as_ft(d["filter"]), "bias": d.get("bias") and as_ft(d["bias"]),
                                  "preluActivationWeights": d.get("preluActivationWeights") and as_ft(d["preluActivationWeights"])},
                         attrs)
            if x3:
                out.squeeze0 = True
                out2 = FT(out.value[0], out.dtype, out.case)
                out2.squeeze0 = True
                return out2
            return out
        return f

    fused = NS()
    fused.conv2d = fused_conv("fused_conv2d")
    fused.depthwiseConv2d = fused_conv("fused_depthwise_conv2d")

    def fused_matmul(d):
        return rec.op("fused_mat_mul",
                      {"a": as_ft(d["a"]), "b": as_ft(d["b"]),
                       "bias": d.get("bias") and as_ft(d["bias"]),
                       "preluActivationWeights": d.get("preluActivationWeights") and as_ft(d["preluActivationWeights"])},
                      {"transposeA": bool(d.get("transposeA")), "transposeB": bool(d.get("transposeB")),
                       "activation": d.get("activation") or "linear",
                       "leakyreluAlpha": d.get("leakyreluAlpha", 0.2) if d.get("leakyreluAlpha") is not None else 0.2})
    fused.matMul = fused_matmul
    tf.fused = fused

    def conv(opname):
        def f(x, filt, strides, pad, dataFormat="NHWC", dilations=None, dimRoundingMode=None):
            if dataFormat not in (None, "NHWC"):
                raise Skip("NCHW")
            x, filt = as_ft(x), as_ft(filt)
            x3 = x.rank == 3
            xx = FT(x.value[None], x.dtype) if x3 else x
            out = rec.op(opname, {"x": xx, "filter": filt},
                         {"strides": strides, "pad": pad, "dilations": dilations or [1, 1],
                          "dimRoundingMode": dimRoundingMode})
            if x3:
                o2 = FT(out.value[0], out.dtype, out.case)
                o2.squeeze0 = True
                return o2
            return out
        return f
    tf.conv2d = conv("conv2d")
    tf.depthwiseConv2d = conv("depthwise_conv2d")

    def matmul(a, b, transposeA=False, transposeB=False):
        a, b = as_ft(a), as_ft(b)
        if a.dtype != "float32" or b.dtype != "float32":
            raise Skip("non-float matmul")
        return rec.op("mat_mul", {"a": a, "b": b},
                      {"transposeA": bool(transposeA), "transposeB": bool(transposeB)})
    tf.matMul = matmul

    def pool(opname):
        def f(x, filterSize, strides, pad, dimRoundingMode=None):
            x = as_ft(x)
            if x.dtype != "float32":
                raise Skip("int pool")
            x3 = x.rank == 3
            xx = FT(x.value[None], x.dtype) if x3 else x
            out = rec.op(opname, {"x": xx}, {"filterSize": filterSize, "strides": strides,
                                             "pad": pad, "dimRoundingMode": dimRoundingMode})
            if x3:
                o2 = FT(out.value[0], out.dtype, out.case)
                o2.squeeze0 = True
                return o2
            return out
        return f
    tf.maxPool = pool("max_pool")
    tf.avgPool = pool("avg_pool")

    def unary(opname):
        def f(x):
            x = as_ft(x)
            if x.dtype != "float32":
                raise Skip("non-float unary")
            return rec.op(opname, {"x": x}, {})
        return f
    for js, py in (("relu", "relu"), ("relu6", "relu6"), ("elu", "elu"), ("sigmoid", "sigmoid"),
                   ("exp", "exp"), ("sqrt", "sqrt"), ("rsqrt", "rsqrt"), ("square", "square"),
                   ("tanh", "tanh"), ("neg", "neg"), ("erf", "erf"), ("abs", "abs"), ("log", "log")):
        setattr(tf, js, unary(py))

    def leaky(x, alpha=0.2):
        x = as_ft(x)
        if x.dtype != "float32":
            raise Skip("non-float unary")
        return rec.op("leaky_relu", {"x": x}, {"alpha": alpha})
    tf.leakyRelu = leaky

    def clip(x, lo, hi):
        x = as_ft(x)
        if x.dtype != "float32":
            raise Skip("non-float clip")
        return rec.op("clip_by_value", {"x": x}, {"lo": lo, "hi": hi})
    tf.clipByValue = clip

    def prelu(x, alpha):
        return rec.op("prelu", {"x": as_ft(x), "alpha": as_ft(alpha)}, {})
    tf.prelu = prelu

    def binary(opname):
        def f(a, b):
            a, b = as_ft(a), as_ft(b)
            if a.dtype != b.dtype or a.dtype == "bool":
                raise Skip("mixed dtype binary")
            return rec.op(opname, {"a": a, "b": b}, {}, a.dtype)
        return f
    for js, py in (("add", "add"), ("sub", "sub"), ("mul", "mul"), ("maximum", "maximum"),
                   ("minimum", "minimum"), ("squaredDifference", "squared_difference")):
        setattr(tf, js, binary(py))

    def softmax(x, dim=-1):
        return rec.op("softmax", {"logits": as_ft(x)}, {"dim": dim})
    tf.softmax = softmax

    def reduce(opname):
        def f(x, axis=None, keepDims=False):
            x = as_ft(x)
            if x.dtype != "float32":
                raise Skip("non-float reduce")
            return rec.op(opname, {"x": x}, {"axis": axis, "keepDims": bool(keepDims)})
        return f
    tf.sum, tf.mean, tf.max = reduce("sum"), reduce("mean"), reduce("max")

    def argmax(x, axis=0):
        x = as_ft(x)
        if x.dtype != "float32":
            raise Skip("non-float argmax")
        return rec.op("arg_max", {"x": x}, {"axis": axis}, "int32")
    tf.argMax = argmax

    def transpose(x, perm=None):
        x = as_ft(x)
        return rec.op("transpose", {"x": x}, {"perm": perm}, x.dtype)
    tf.transpose = transpose

    def gather(x, indices, axis=0, batchDims=0):
        x, indices = as_ft(x), as_ft(indices, "int32")
        if indices.dtype != "int32":
            indices = FT(indices.value.astype(np.int32), "int32")
        return rec.op("gather", {"x": x, "indices": indices}, {"axis": axis, "batchDims": batchDims},
                      x.dtype)
    tf.gather = gather

    def tile(x, reps):
        x = as_ft(x)
        return rec.op("tile", {"x": x}, {"reps": list(reps)}, x.dtype)
    tf.tile = tile

    def batchnorm(x, mean, variance, offset=None, scale=None, varianceEpsilon=None):
        return rec.op("batch_norm", {"x": as_ft(x), "mean": as_ft(mean), "variance": as_ft(variance),
                                     "offset": offset is not None and as_ft(offset) or None,
                                     "scale": scale is not None and as_ft(scale) or None},
                      {"varianceEpsilon": varianceEpsilon})
    tf.batchNorm = tf.batchNorm2d = tf.batchNorm3d = tf.batchNorm4d = batchnorm

    tf.pow = binary("pow")
    real_div = binary("div")

    def div(a, b):
        a, b = as_ft(a), as_ft(b)
        if a.dtype == "int32" and b.dtype == "int32":
            raise Skip("int32 div is the FloorDiv kernel")      # tfjs-core/src/ops/div.ts:55-57
        return real_div(a, b)
    tf.div = div

    def dot(t1, t2):
        """tfjs-core/src/ops/dot.ts:45-72: vectors become 1 x n / n x 1 matrices."""
        t1, t2 = as_ft(t1), as_ft(t2)
        if t1.rank == 1 and t2.rank == 1:
            return matmul(t1.reshape([1, -1]), t2.reshape([-1, 1])).reshape([])
        if t1.rank == 1 and t2.rank == 2:
            return matmul(t1.reshape([1, -1]), t2).reshape([-1])
        if t1.rank == 2 and t2.rank == 1:
            return matmul(t1, t2.reshape([-1, 1])).reshape([-1])
        return matmul(t1, t2)
    tf.dot = dot
    tf.outerProduct = lambda v1, v2: matmul(as_ft(v1).reshape([-1, 1]), as_ft(v2).reshape([1, -1]))

    def cast(x, dtype):
        x = as_ft(x)
        if dtype not in ("float32", "int32", "bool"):
            raise Skip("dtype %s" % dtype)
        return rec.op("cast", {"x": x}, {"dtype": dtype}, dtype)
    tf.cast = cast

    def same_dtype(ts):
        ts = [as_ft(t) for t in ts]
        if len(set(t.dtype for t in ts)) != 1:
            raise Skip("mixed dtype")
        return ts

    def chained_list(tensors, rest):
        """a.concat(b, axis) / a.stack(b, axis): (tensor list, axis)."""
        if isinstance(tensors, FT):
            other = rest[0] if rest else []
            tensors = [tensors] + (list(other) if isinstance(other, (list, tuple)) else [other])
            rest = rest[1:]
        return tensors, (rest[0] if rest else 0)

    def concat(tensors, *rest, **kw):
        tensors, axis = chained_list(tensors, rest)
        axis = kw.get("axis", axis)
        ts = same_dtype(tensors)
        return rec.op("concat", {"tensors": ts}, {"axis": axis}, ts[0].dtype)
    tf.concat = tf.concat1d = tf.concat2d = tf.concat3d = tf.concat4d = concat

    def stack(tensors, *rest, **kw):
        tensors, axis = chained_list(tensors, rest)
        axis = kw.get("axis", axis)
        ts = same_dtype(tensors)
        return rec.op("stack", {"tensors": ts}, {"axis": axis}, ts[0].dtype)
    tf.stack = stack

    def expand_dims(x, axis=0):
        x = as_ft(x)
        return rec.op("expand_dims", {"x": x}, {"axis": axis}, x.dtype)
    tf.expandDims = expand_dims

    def slice_(x, begin, size=None):
        x = as_ft(x)
        return rec.op("slice", {"x": x}, {"begin": begin, "size": size}, x.dtype)
    tf.slice = tf.slice1d = tf.slice2d = tf.slice3d = tf.slice4d = slice_

    def pad(x, paddings, constantValue=0):
        x = as_ft(x)
        if x.rank == 1 and paddings and not isinstance(paddings[0], (list, tuple)):
            paddings = [paddings]      # pad1d takes one [before, after] pair
        return rec.op("pad", {"x": x}, {"paddings": [list(p) for p in paddings],
                                        "constantValue": constantValue}, x.dtype)
    tf.pad = tf.pad1d = tf.pad2d = tf.pad3d = tf.pad4d = pad

    tf.memory = lambda: Obj({"numTensors": 0, "numDataBuffers": 0, "numBytes": 0})
    tf.engine = lambda: Obj({"backend": Obj({"numDataIds": lambda: 0})})
    tf.dispose = lambda *a: None
    tf.backend = lambda: Obj({"floatPrecision": lambda: 32})
    FT.tf = tf
    return tf


def file_helpers(src):
    """Python source for the file-level `function name(args) {...}` helpers."""
    out = []
    for m in re.finditer(r"(?m)^function\s+(\w+)\s*\(([^)]*)\)\s*(?::[^{]+)?\{", src):
        brace = m.end() - 1
        try:
            close = match_close(src, brace)
            params = [re.match(r"\s*(\w+)", p).group(1) for p in m.group(2).split(",") if p.strip()]
            body = tr_block(src[brace + 1:close], 1)
        except (Skip, AttributeError):
            continue
        out.append("def %s(%s):\n%s" % (m.group(1), ", ".join(params), "\n".join(body or ["    pass"])))
    return "\n".join(out)


def generate_case_inputs(total_tensor, total_filter):
    """fused_conv2d_test.ts:22-35 / conv2d_test.ts helper of the same name."""
    inp = [i * 0.001 - total_tensor * 0.001 / 2 for i in range(int(total_tensor))]
    filt = [i * 0.001 * (-1 if i % 2 == 0 else 1) for i in range(int(total_filter))]
    class CaseInputs(object):
        pass
    out = CaseInputs()
    out.input, out.filter = inp, filt
    return out


def optimal_window(n):
    if n <= 30:
        return n
    a = int(math.floor(math.sqrt(n)))
    while a < n:
        if n % a == 0:
            return a
        a += 1
    return n


def set_index(lst, i, v):
    i = int(i)
    if i >= len(lst):
        lst.extend([None] * (i + 1 - len(lst)))
    lst[i] = v


class Obj(object):
    def __init__(self, d):
        self.__dict__.update(d)


def run_spec(py_lines, rec, goldens_out, meta, helpers=""):
    checks = []

    def close(actual, expected, eps=None):
        if not isinstance(actual, Data):
            raise Skip("expectArraysClose on non-tensor data")
        if isinstance(expected, Data):
            raise Skip("expected is tensor data")
        checks.append((actual.t, np.asarray(expected, np.float64).reshape(-1)))

    def expect_equal(a, b):
        pass

    env = {"tf": make_tf(rec), "expectArraysClose": close, "expectArraysEqual": close,
           "__expect_equal": expect_equal, "__nan": float("nan"), "__inf": float("inf"),
           "__math": math, "__typed": lambda v: list(v) if not isinstance(v, (int, float)) else [0] * int(v),
           "__newarray": lambda n=0: [None] * int(n), "generateCaseInputs": generate_case_inputs,
           "dict": dict, "len": len, "range": range, "int": int,
           "MATMUL_SHARED_DIM_THRESHOLD": 1000,  # mat_mul_test.ts:24
           "__obj": Obj, "__setidx": set_index,
           # tfjs-core/src/util_base.ts tanh (Math.tanh with the overflow guards)
           "util": Obj({"tanh": math.tanh}),
           # reduce_util.ts:24-38 with nearestDivisor of util_base.ts
           "reduce_util": Obj({"PARALLELIZE_THRESHOLD": 30,
                               "computeOptimalWindowSize": optimal_window}),
           "env": Obj({"backendName": "cpu"}), "__arrayfrom": lambda v: v,
           "backend": lambda: Obj({"floatPrecision": lambda: 32})}
    if helpers:
        exec(helpers, env)
    # the spec body runs as a function so that an early `return` is legal
    exec("def __spec():\n" + "\n".join("    " + ln for ln in (py_lines or ["pass"])) +
         "\n__spec()\n", env)
    for t, expected in checks:
        if t.case is None:
            continue
        case = t.case
        goldens_out.append(dict(meta, op=case["op"], inputs=case["inputs"], attrs=case["attrs"],
                                input_dtypes=case["input_dtypes"], expected=expected,
                                expected_shape=list(getattr(t, "op_shape", t.value.shape)),
                                squeeze0=bool(getattr(t, "squeeze0", False))))


def to_jsonable(v):
    if isinstance(v, np.ndarray):
        def enc(x):
            x = float(x)
            if math.isnan(x):
                return "NaN"
            if math.isinf(x):
                return "Infinity" if x > 0 else "-Infinity"
            return x
        return {"shape": list(v.shape), "dtype": str(v.dtype),
                "data": [enc(x) for x in v.reshape(-1).tolist()]}
    if isinstance(v, dict):
        return {k: to_jsonable(x) for k, x in v.items()}
    if isinstance(v, (list, tuple)):
        return [to_jsonable(x) for x in v]
    if isinstance(v, (np.integer,)):
        return int(v)
    if isinstance(v, (np.floating,)):
        return float(v)
    return v


def main(ref_root, out_path):
    goldens, summary = [], {}
    for rel in TEST_FILES:
        path = os.path.join(ref_root, rel)
        if not os.path.exists(path):
            summary[rel] = {"missing": True}
            continue
        src = strip_comments(open(path).read())
        stats = {"specs": 0, "extracted_specs": 0, "cases": 0, "skipped": {}}
        helpers = file_helpers(src)
        setups = find_setups(src)
        for name, line, body, pos in find_specs(src):
            stats["specs"] += 1
            body = "".join(b + ";\n" for a, e, b in sorted(setups) if a < pos < e) + body
            before = len(goldens)
            try:
                if re.search(r"\btf\.(grad|grads|valueAndGrad|customGrad|complex|browser)\b", body):
                    raise Skip("gradient / complex / browser")
                if "toThrow" in body or "rejects" in body:
                    raise Skip("error-path spec")
                py = tr_block(body)
                run_spec(py, Recorder(), goldens, {"file": rel, "line": line, "spec": name},
                         helpers)
            except Skip as e:
                del goldens[before:]
                key = str(e).split(":")[0][:40]
                stats["skipped"][key] = stats["skipped"].get(key, 0) + 1
                continue
            except Exception as e:  # translation gap: count it, keep going
                del goldens[before:]
                key = "translator: %s" % type(e).__name__
                msg = str(e)
                if isinstance(e, ValueError) and "could not convert string" in msg:
                    key = "string tensor"
                elif isinstance(e, AttributeError) and "'NS' object has no attribute" in msg:
                    key = "op outside the hot path"   # tf.mod, tf.atan2, tf.squeeze ...
                elif isinstance(e, NameError) and "encodeString" in msg:
                    key = "string tensor"
                stats["skipped"][key] = stats["skipped"].get(key, 0) + 1
                continue
            if len(goldens) > before:
                stats["extracted_specs"] += 1
                stats["cases"] += len(goldens) - before
        summary[rel] = stats
    # keep the fixture small: drop cases with very large tensors
    kept = []
    for g in goldens:
        n = sum(np.asarray(v).size if not isinstance(v, list) else sum(np.asarray(t).size for t in v)
                for v in g["inputs"].values()) + g["expected"].size
        if n <= 20000:
            kept.append(g)
    with open(out_path, "w") as f:
        json.dump({"summary": summary, "cases": [to_jsonable(g) for g in kept]}, f,
                  separators=(",", ":"))
    total = sum(s.get("cases", 0) for s in summary.values())
    print("extracted %d cases (%d kept) from %d files -> %s" %
          (total, len(kept), len(TEST_FILES), out_path))
    for rel, s in summary.items():
        print("  %-62s specs %3d  extracted %3d  cases %3d  skipped %s" %
              (rel, s.get("specs", 0), s.get("extracted_specs", 0), s.get("cases", 0),
               s.get("skipped", s)))


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: %s <path to a tensorflow/tfjs checkout> [output file]" % sys.argv[0])
    main(sys.argv[1],
         sys.argv[2] if len(sys.argv) > 2 else os.path.join(ROOT, "tests", "golden", "ts_goldens.json"))
