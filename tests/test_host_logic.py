"""Host-side logic that needs no GPU: canonical form of elementwise chains, the chain
catalogue query of the library, leaf addressing modes, batch sharding."""
import ctypes

import numpy as np
import pytest

from tfjs_b200 import _cabi
from tfjs_b200.backend import PendingEw, _canonical_program

ADD, SUB, MUL, DIV = (_cabi.BINARY_OPS[n] for n in ("Add", "Sub", "Multiply", "RealDiv"))
ERF = _cabi.EW_UNARY + _cabi.UNARY_OPS["Erf"]
RELU = _cabi.EW_UNARY + _cabi.UNARY_OPS["Relu"]
FULL, PER, ROW, SCAL, BAT = (_cabi.EW_FULL, _cabi.EW_PERIODIC, _cabi.EW_ROW, _cabi.EW_SCALAR,
                             _cabi.EW_BATCHED)


def _signature(ops, modes):
    c_ops, order = _canonical_program(ops, modes)
    slot = lambda r: r[1] if r[0] == "in" else len(order) + r[1]
    return [(code, slot(a), slot(b)) for code, a, b in c_ops], [modes[k] for k in order]


def _gelu(order):
    """x * 0.5 * (1 + erf(x * c)) written with the operands of every commutative op in the
    given order; leaves: 0 x, 1 half, 2 c, 3 one."""
    sw = (lambda a, b: (b, a)) if order else (lambda a, b: (a, b))
    return [(MUL,) + sw(("in", 0), ("in", 1)), (MUL,) + sw(("in", 0), ("in", 2)),
            (ERF, ("op", 1), ("op", 1)), (ADD,) + sw(("op", 2), ("in", 3)),
            (MUL,) + sw(("op", 0), ("op", 3))]


def test_canonical_program_ignores_operand_order_of_commutative_ops():
    a = _signature(_gelu(False), [FULL, SCAL, SCAL, SCAL])
    b = _signature(_gelu(True), [FULL, SCAL, SCAL, SCAL])
    assert a == b
    assert a[0] == [(MUL, 0, 1), (ERF, 4, 4), (ADD, 5, 2), (MUL, 0, 3), (MUL, 6, 7)]
    # Sub is not commutative: its operand order survives
    s1 = _signature([(SUB, ("in", 0), ("in", 1))], [FULL, ROW])
    s2 = _signature([(SUB, ("in", 1), ("in", 0))], [FULL, ROW])
    assert s1[0] == [(SUB, 0, 1)] and s2[0] == [(SUB, 0, 1)] and s1[1] != s2[1]


def test_canonical_program_emits_a_shared_value_once():
    # (a + b) used twice: relu(s) * s
    ops = [(ADD, ("in", 0), ("in", 1)), (RELU, ("op", 0), ("op", 0)), (MUL, ("op", 1), ("op", 0))]
    sig, _ = _signature(ops, [FULL, FULL])
    assert len(sig) == 3 and sum(1 for code, _, _ in sig if code == ADD) == 1


CHAINS = {
    "layer_norm_tail": ([(SUB, ("in", 0), ("in", 1)), (MUL, ("op", 0), ("in", 2)),
                         (MUL, ("op", 1), ("in", 3)), (ADD, ("op", 2), ("in", 4))],
                        [FULL, ROW, ROW, PER, PER], True),
    "layer_norm_tail_bn": ([(MUL, ("in", 1), ("in", 2)), (MUL, ("in", 0), ("op", 0)),
                            (MUL, ("in", 1), ("in", 2)), (MUL, ("in", 4), ("op", 2)),
                            (SUB, ("in", 3), ("op", 3)), (ADD, ("op", 1), ("op", 4))],
                           [FULL, ROW, PER, PER, ROW], True),
    "gelu_mul": (_gelu(False), [FULL, SCAL, SCAL, SCAL], True),
    "gelu_div": ([(MUL, ("in", 0), ("in", 1)), (DIV, ("in", 0), ("in", 2)),
                  (ERF, ("op", 1), ("op", 1)), (ADD, ("op", 2), ("in", 3)),
                  (MUL, ("op", 0), ("op", 3))], [FULL, SCAL, SCAL, SCAL], True),
    "scale_mask": ([(MUL, ("in", 0), ("in", 1)), (ADD, ("op", 0), ("in", 2))],
                   [FULL, SCAL, BAT], True),
    "add_add": ([(ADD, ("in", 0), ("in", 1)), (ADD, ("op", 0), ("in", 2))],
                [FULL, FULL, PER], True),
    "not_catalogued": ([(SUB, ("in", 0), ("in", 1)), (RELU, ("op", 0), ("op", 0))],
                       [FULL, FULL], False),
}


@pytest.mark.parametrize("name", sorted(CHAINS))
def test_library_catalogue_knows_the_chains_of_the_graph_models(name):
    """The canonical programs the host layer builds for the decomposed LayerNorm, GELU and
    score scaling are the ones the library has straight-line kernels for (the query needs
    no GPU and no context state)."""
    ops, modes, expected = CHAINS[name]
    sig, _ = _signature(ops, modes)
    prog = _cabi.EwProgram()
    prog.n_inputs, prog.n_ops = len(modes), len(sig)
    for j, (code, a, b) in enumerate(sig):
        prog.ops[j].opcode, prog.ops[j].a, prog.ops[j].b = code, a, b
    lib = _cabi.load()
    yes = ctypes.c_int32(-1)
    # the query reads the program only; a dummy non-null context pointer is never followed
    dummy = ctypes.create_string_buffer(8)
    rc = lib.tfjs_cuda_fused_elementwise_catalogued(ctypes.cast(dummy, ctypes.c_void_p),
                                                    ctypes.byref(prog), ctypes.byref(yes))
    assert rc == _cabi.OK
    assert bool(yes.value) == expected


def test_leaf_addressing_modes():
    p = PendingEw([], [], [], [4, 12, 16, 32], [], (ADD, None, [1], None, [1]))
    assert p._leaf_mode([4, 12, 16, 32])[0] == FULL
    assert p._leaf_mode([1])[0] == SCAL and p._leaf_mode([])[0] == SCAL
    assert p._leaf_mode([32]) == (PER, 32, 0)
    assert p._leaf_mode([16, 32]) == (PER, 512, 0)
    assert p._leaf_mode([4, 12, 16, 1])[0] == ROW
    assert p._leaf_mode([4, 1, 1, 32]) == (BAT, 32, 12 * 16 * 32)
    assert p._leaf_mode([4, 1, 16, 32]) == (BAT, 512, 12 * 512)
    assert p._leaf_mode([4, 12, 1, 32]) == (BAT, 32, 16 * 32)
    assert p._leaf_mode([1, 12, 1, 32]) is None          # two separate broadcast gaps
    assert p._leaf_mode([1, 12, 1, 1]) is None
    q = PendingEw([], [], [], [8, 1], [], (ADD, None, [1], None, [1]))
    assert q._leaf_mode([8, 1])[0] == FULL and q._leaf_mode([1])[0] == SCAL


# ------------------------------------------------ plan rewrite: layer normalisation --
def _bert_plan():
    import bench
    from tfjs_b200 import graph_model as G
    mj, wt = bench.build_model("bert", 2)
    consts, off = {}, 0
    for group in mj["weightsManifest"]:
        for spec in group["weights"]:
            assert "quantization" not in spec
            n = int(np.prod(spec["shape"])) if spec["shape"] else 1
            consts[spec["name"]] = np.frombuffer(
                wt, dtype=np.dtype(spec["dtype"]), count=n, offset=off).reshape(spec["shape"])
            off += n * 4
    nodes = [G.Node(d) for d in mj["modelTopology"]["node"]]
    return G, nodes, consts


def _fuse(G, nodes, consts, protected=()):
    return G.fuse_layer_norms(nodes, lambda n: n in consts, lambda n: consts[n].reshape(-1),
                              lambda n: list(consts[n].shape), protected)


def test_layer_norm_subgraphs_of_bert_are_replaced():
    G, nodes, consts = _bert_plan()
    new, n = _fuse(G, nodes, consts)
    assert n == 25                         # embeddings + 2 per encoder layer
    # nine nodes become one, and the Add in front of each (24 residual connections and
    # the sum of the two embeddings) is absorbed
    assert len(new) == len(nodes) - 9 * n
    fused = [x for x in new if x.op == "_FusedLayerNorm"]
    assert len(fused) == n
    names = set(x.name for x in new)
    for f in fused:
        assert len(f.inputs) == 4 and G.attr_bool(f.attrs, "residual")
        assert abs(G.attr_number(f.attrs, "epsilon") - 1e-12) < 1e-18
        assert all(G.parse_node_name(i)[0] in names for i in f.inputs)
    # still topologically ordered
    pos = {x.name: i for i, x in enumerate(new)}
    for x in new:
        for i in x.inputs:
            assert pos[G.parse_node_name(i)[0]] < pos[x.name]
    assert not any(x.op in ("SquaredDifference", "Rsqrt") for x in new)
    # a residual sum that something else reads as well stays a node of its own
    res_sum = next(x for x in nodes if x.op == "AddV2" and x.name not in names and
                   x.inputs == fused[-1].inputs[:2])
    tap = G.Node({"name": "tap", "op": "Identity", "input": [res_sum.name]})
    new2, n2 = _fuse(G, nodes + [tap], consts)
    assert n2 == 25 and any(x.name == res_sum.name for x in new2)
    assert sum(1 for x in new2 if x.op == "_FusedLayerNorm" and len(x.inputs) == 3) == 1


def test_layer_norm_is_left_alone_when_an_intermediate_is_wanted():
    G, nodes, consts = _bert_plan()
    rs = [x for x in nodes if x.op == "Rsqrt"]
    new, n = _fuse(G, nodes, consts, protected=[rs[3].name])
    assert n == 24 and any(x.name == rs[3].name for x in new)
    # a second consumer of the variance keeps that subgraph too
    var = next(x for x in nodes if x.name == G.parse_node_name(
        next(y for y in nodes if y.name == G.parse_node_name(rs[0].inputs[0])[0]).inputs[0])[0])
    extra = G.Node({"name": "tap", "op": "Identity", "input": [var.name]})
    new, n = _fuse(G, nodes + [extra], consts)
    assert n == 24


def test_layer_norm_match_needs_the_last_axis_and_keep_dims():
    G, nodes, consts = _bert_plan()
    mean = next(x for x in nodes if x.op == "Mean")
    consts2 = dict(consts)
    consts2[G.parse_node_name(mean.inputs[1])[0]] = np.array([1], np.int32)
    _, n = _fuse(G, nodes, consts2)
    assert n < 25


# ---------------------------------------------------- plan rewrite: attention heads --
def test_heads_split_and_merge_of_bert_become_store_orders():
    G, nodes, consts = _bert_plan()
    new, n = G.fuse_attention_heads(nodes, lambda x: x in consts, lambda x: consts[x].reshape(-1))
    assert n == 12 * 4                       # Q, K, V splits and one merge per layer
    assert len(new) == len(nodes) - 2 * n    # Reshape + Transpose folded into each product
    assert not any(x.op == "Transpose" for x in new)
    fused = [x for x in new if x.op == "_MatMulHeads"]
    kinds = [G.attr_string(x.attrs, "_layout") for x in fused]
    assert kinds.count("split") == 36 and kinds.count("merge") == 12
    for x in fused:
        inner = G.attr_string(x.attrs, "_op", keep_case=True)
        dims = G.attr_number_list(x.attrs, "_dims")
        if G.attr_string(x.attrs, "_layout") == "split":
            assert inner == "_FusedMatMul" and dims == [2, 128, 12, 64] and len(x.inputs) == 3
        else:
            assert inner == "BatchMatMulV2" and dims == [256, 768] and len(x.inputs) == 2
    pos = {x.name: i for i, x in enumerate(new)}
    for x in new:
        for i in x.inputs:
            assert pos[G.parse_node_name(i)[0]] < pos[x.name]
    # both rewrites together, as the executor applies them
    both, k = _fuse(G, new, consts)
    assert k == 25


def test_heads_rewrite_keeps_a_product_that_is_read_elsewhere():
    G, nodes, consts = _bert_plan()
    t = next(x for x in nodes if x.op == "Transpose")
    r = next(x for x in nodes if x.name == G.parse_node_name(t.inputs[0])[0])
    tap = G.Node({"name": "tap", "op": "Identity", "input": [r.inputs[0]]})
    new, n = G.fuse_attention_heads(nodes + [tap], lambda x: x in consts,
                                    lambda x: consts[x].reshape(-1))
    assert n == 47 and any(x.name == t.name and x.op == "Transpose" for x in new)
    _, n = G.fuse_attention_heads(nodes, lambda x: x in consts, lambda x: consts[x].reshape(-1),
                                  protected=[r.name])
    assert n == 47


# ------------------------------------------------- plan rewrite: softmax of scores --
def test_scaled_masked_softmax_of_bert_is_one_node():
    G, nodes, consts = _bert_plan()
    new, n = G.fuse_softmax_inputs(nodes, lambda x: x in consts, lambda x: consts[x].reshape(-1))
    assert n == 12 and len(new) == len(nodes) - 2 * n
    for x in new:
        if x.op == "_SoftmaxScaledMasked":
            assert len(x.inputs) == 2
            assert abs(G.attr_number(x.attrs, "_scale") - float(np.float32(0.125))) < 1e-12
    sm = next(x for x in nodes if x.op == "Softmax")
    _, n = G.fuse_softmax_inputs(nodes, lambda x: x in consts, lambda x: consts[x].reshape(-1),
                                 protected=[G.parse_node_name(sm.inputs[0])[0]])
    assert n == 11


# --------------------------------------------- plan rewrite: one node per attention --
def test_attention_of_bert_becomes_one_node_per_layer():
    G, nodes, consts = _bert_plan()
    is_const, value = (lambda x: x in consts), (lambda x: consts[x].reshape(-1))
    heads, k = G.fuse_attention_heads(nodes, is_const, value)
    soft, j = G.fuse_softmax_inputs(heads, is_const, value)
    new, n = G.fuse_attention(soft)
    assert (k, j, n) == (48, 12, 12)
    assert len(new) == len(soft) - 2 * n         # scores and probabilities are gone
    by_name = {x.name: x for x in new}
    for x in new:
        assert x.op not in ("BatchMatMul", "BatchMatMulV2", "Softmax", "_SoftmaxScaledMasked")
        if x.op != "_FusedAttention":
            continue
        assert len(x.inputs) == 4                # q, k, v, mask
        for i in x.inputs[:3]:                   # the three heads-split projections
            assert by_name[G.parse_node_name(i)[0]].op == "_MatMulHeads"
        assert abs(G.attr_number(x.attrs, "_scale") - 0.125) < 1e-12
        assert G.attr_number_list(x.attrs, "_dims") == [256, 768]
    pos = {x.name: i for i, x in enumerate(new)}
    for x in new:
        for i in x.inputs:
            assert pos[G.parse_node_name(i)[0]] < pos[x.name]
    # scores that something else reads stay
    sc = next(x for x in soft if x.op in ("BatchMatMul", "BatchMatMulV2"))
    tap = G.Node({"name": "tap", "op": "Identity", "input": [sc.name]})
    _, n = G.fuse_attention(soft + [tap])
    assert n == 11
    _, n = G.fuse_attention(soft, protected=[sc.name])
    assert n == 11
    # without the softmax rewrite the Mul / AddV2 sit between the product and the softmax
    _, n = G.fuse_attention(heads)
    assert n == 0


def test_softmax_mask_rows():
    from tfjs_b200.kernels.reduce import softmax_mask_rows as f
    assert f([64, 12, 128, 128], [64, 1, 1, 128]) == 12 * 128
    assert f([64, 12, 128, 128], [64, 12, 128, 128]) == 1
    assert f([64, 12, 128, 128], [128]) == 64 * 12 * 128
    assert f([64, 12, 128, 128], [1, 1, 1, 128]) == 64 * 12 * 128
    assert f([64, 12, 128, 128], [64, 12, 1, 128]) == 128
    assert f([64, 12, 128, 128], [1, 12, 1, 128]) is None
    assert f([64, 12, 128, 128], [64, 1, 128, 128]) is None
    assert f([64, 12, 128, 128], [64, 1, 1, 1]) is None
    assert f([5, 7], [7]) == 5 and f([7], [7]) == 1


# ------------------------------------------------------ plan rewrite: erf GELU --
def test_erf_gelu_after_a_dense_layer_becomes_its_epilogue():
    G, nodes, consts = _bert_plan()
    new, n = G.fuse_gelu_into_matmul(nodes, lambda x: x in consts, lambda x: consts[x].reshape(-1))
    assert n == 12 and len(new) == len(nodes) - 5 * n
    assert not any(x.op == "Erf" for x in new)
    for x in new:
        if x.op == "_FusedMatMulGelu":
            p = G.attr_number_list(x.attrs, "_gelu")
            assert len(x.inputs) == 3
            assert p == [float(np.float32(1 / np.sqrt(2.0))), 0.5, 1.0, 0.0]
    # the dense output read by something else keeps the five nodes
    erf = next(x for x in nodes if x.op == "Erf")
    mul = next(x for x in nodes if x.name == G.parse_node_name(erf.inputs[0])[0])
    h = next(i for i in mul.inputs if G.parse_node_name(i)[0] not in consts)
    tap = G.Node({"name": "tap", "op": "Identity", "input": [h]})
    _, n = G.fuse_gelu_into_matmul(nodes + [tap], lambda x: x in consts,
                                   lambda x: consts[x].reshape(-1))
    assert n == 11


def test_manifest_entry_checks_follow_decode_weight():
    """The loader's per-entry validation (storage kind, element count, stored bytes) and
    the reference's error cases (tfjs-core/src/io/io_utils.ts:196-218, :269-272)."""
    from tfjs_b200 import _cabi, io
    e = io._entry({"name": "w", "shape": [3, 4], "dtype": "float32"})
    assert e == (_cabi.STORED_RAW, "float32", 12, 48)
    e = io._entry({"name": "w", "shape": [5], "dtype": "bool"})
    assert e == (_cabi.STORED_RAW, "bool", 5, 5)
    e = io._entry({"name": "w", "shape": [2, 5], "dtype": "int32",
                   "quantization": {"dtype": "uint16", "scale": 1.0, "min": 0.0}})
    assert e == (_cabi.STORED_UINT16, "int32", 10, 20)
    e = io._entry({"name": "w", "shape": [7], "dtype": "float32", "quantization": {"dtype": "float16"}})
    assert e == (_cabi.STORED_FLOAT16, "float32", 7, 14)
    import pytest
    with pytest.raises(ValueError, match="doesn't have corresponding metadata"):
        io._entry({"name": "w", "shape": [1], "dtype": "float32", "quantization": {"dtype": "uint8"}})
    with pytest.raises(ValueError, match="only supports weights of type float32"):
        io._entry({"name": "w", "shape": [1], "dtype": "int32", "quantization": {"dtype": "float16"}})
    with pytest.raises(ValueError, match="unknown quantization dtype"):
        io._entry({"name": "w", "shape": [1], "dtype": "float32",
                   "quantization": {"dtype": "uint4", "scale": 1, "min": 0}})
    with pytest.raises(ValueError, match="string weights"):
        io._entry({"name": "w", "shape": [1], "dtype": "string"})
    with pytest.raises(ValueError, match="Unsupported dtype"):
        io._entry({"name": "w", "shape": [1], "dtype": "complex64"})


def test_hoist_keeps_the_plan_topological_and_groups_projections():
    """hoist_shared_operand_matmuls moves the products that read one tensor next to each
    other (with their constants) without breaking the order of dependencies."""
    from tfjs_b200 import graph_model, model_zoo
    from tfjs_b200.graph_model import parse_node_name
    model_json, _ = model_zoo.bert_encoder(2)
    nodes = [graph_model.Node(n) for n in model_json["modelTopology"]["node"]]
    consts = set(n.name for n in nodes if n.op == "Const")
    out, moved = graph_model.hoist_shared_operand_matmuls(nodes, lambda name: name in consts)
    assert moved > 0 and sorted(n.name for n in out) == sorted(n.name for n in nodes)
    seen = set()
    for n in out:
        for i in n.inputs:
            assert parse_node_name(i)[0] in seen, (n.name, i)
        seen.add(n.name)
    # every layer's query, key and value projections: three products in a row on one operand
    pos = {n.name: k for k, n in enumerate(out)}
    by_a = {}
    for n in out:
        if n.op == "_FusedMatMul":
            by_a.setdefault(n.inputs[0], []).append(n)
    triples = [v for v in by_a.values() if len(v) == 3]
    assert len(triples) == 12
    for v in triples:
        inner = [x for x in out[pos[v[0].name]:pos[v[2].name] + 1] if x.op != "Const"]
        assert [x.name for x in inner] == [x.name for x in v]
