"""_FusedMatMul and BatchMatMul.

Reference kernels: tfjs-backend-cpu/src/kernels/_FusedMatMul.ts:26-62 and
BatchMatMul.ts:25-133 (any rank >= 2, outer dimensions broadcast, operand
batches wrap with `bi % batchDim`).
"""
from ctypes import byref

import numpy as np

from .. import _cabi
from ..backend import PendingMatMul
from ..kernel_registry import KernelConfig
from ..util import assert_and_get_broadcast_shape, size_from_shape
from .common import BACKEND, assert_not_complex, dev, per_channel_len, require_float32
from . import elementwise


def _matmul_impl(backend, a, b, transpose_a, transpose_b, bias, prelu, activation, alpha,
                 heads=None, gelu=None):
    """heads: None, or (layout, rows_or_heads, head_dim, out_shape) for the product stored
    through the heads permutation (tfjs_cuda_fused_matmul_heads); bias and activation must
    then be fusable, and a refusal by the library propagates as CudaError(UNSUPPORTED)."""
    assert_not_complex([a, b], "matMul")
    require_float32(a, "matMul")
    require_float32(b, "matMul")
    a_rank, b_rank = len(a.shape), len(b.shape)
    if a_rank < 2 or b_rank < 2:
        raise ValueError("Error in matMul: inputs must have at least rank 2, got ranks "
                         "%d and %d." % (a_rank, b_rank))
    inner_a = a.shape[a_rank - 2] if transpose_a else a.shape[a_rank - 1]
    inner_b = b.shape[b_rank - 1] if transpose_b else b.shape[b_rank - 2]
    outer_a = a.shape[a_rank - 1] if transpose_a else a.shape[a_rank - 2]
    outer_b = b.shape[b_rank - 2] if transpose_b else b.shape[b_rank - 1]
    outer_dims_a, outer_dims_b = a.shape[:-2], b.shape[:-2]
    batch_a, batch_b = size_from_shape(outer_dims_a), size_from_shape(outer_dims_b)
    out_outer = assert_and_get_broadcast_shape(outer_dims_a, outer_dims_b)
    out_shape = out_outer + [outer_a, outer_b]
    if inner_a != inner_b:
        raise ValueError(
            "Error in matMul: inner shapes (%d) and (%d) of Tensors with shapes %s and %s "
            "and transposeA=%s and transposeB=%s must match." %
            (inner_a, inner_b, ",".join(map(str, a.shape)), ",".join(map(str, b.shape)),
             str(bool(transpose_a)).lower(), str(bool(transpose_b)).lower()))
    batch = max(batch_a, batch_b)
    if batch_a == 0 or batch_b == 0 or batch % max(batch_a, 1) or batch % max(batch_b, 1):
        if batch_a != 0 and batch_b != 0:
            raise ValueError("matMul: the CUDA backend needs batch dims where one divides "
                             "the other, got %d and %d" % (batch_a, batch_b))
    bias_len = per_channel_len(bias, outer_b)
    prelu_len = per_channel_len(prelu, outer_b) if activation == "prelu" else 0
    fuse_bias = bias_len is not None
    fuse_act = fuse_bias and (activation != "prelu" or prelu_len is not None)
    if activation == "gelu_erf" and not (fuse_act and gelu is not None):
        # only exists as a fused epilogue (graph_model.fuse_gelu_into_matmul)
        raise _cabi.CudaError(_cabi.UNSUPPORTED, "matMul: gelu_erf needs a fusable bias")
    if heads is not None and not (fuse_bias and fuse_act and size_from_shape(out_shape)):
        raise _cabi.CudaError(_cabi.UNSUPPORTED, "matMul heads: bias / activation not fusable")
    if (backend.lazy_fusion and backend.group_matmuls and fuse_bias and fuse_act and
            batch_a == 1 and batch_b == 1 and not transpose_a and inner_a % 4 == 0 and
            outer_b > 128 and activation not in ("prelu", "gelu_erf") and
            (bias is None or bias_len == outer_b) and
            # a heads-permuted store the library may decline must be refused here, at the
            # call, where the node executor can still fall back to product + Reshape + Transpose
            (heads is None or (heads[0] == _cabi.HEADS_SPLIT and backend.math_mode == "tf32" and
                               heads[1] % 32 == 0 and heads[2] % 32 == 0)) and
            size_from_shape(out_shape)):
        # Deferred: products that share `a` and these dimensions launch as one group when
        # the first of them is needed (the Q, K and V projections of an attention layer).
        p = _cabi.MatMulParams()
        p.batch_a, p.batch_b = 1, 1
        p.m, p.n, p.k = outer_a, outer_b, inner_a
        p.transpose_a, p.transpose_b = 0, int(bool(transpose_b))
        p.activation = _cabi.ACTIVATIONS[activation]
        p.bias_len = bias_len
        p.prelu_len = 0
        p.leakyrelu_alpha = 0.2 if alpha is None else float(alpha)
        shape = out_shape if heads is None else heads[3]
        desc = {"name": "_FusedMatMul" if heads is None else "_MatMulHeads",
                "inputShapes": dict([("a", list(a.shape)), ("b", list(b.shape))] +
                                    ([("bias", list(bias.shape))] if bias is not None else [])),
                "outputShapes": [list(shape)],
                "attrs": {"transposeA": False, "transposeB": bool(transpose_b)}}
        return backend.defer(shape, "float32", PendingMatMul(
            p, a.dataId, b.dataId, bias.dataId if bias is not None else None,
            None if heads is None else tuple(heads[:3]), [desc]))
    out = backend.make_output(out_shape if heads is None else heads[3], "float32")
    if size_from_shape(out_shape) and batch_a and batch_b:
        p = _cabi.MatMulParams()
        p.batch_a, p.batch_b = batch_a, batch_b
        p.m, p.n, p.k = outer_a, outer_b, inner_a
        p.transpose_a, p.transpose_b = int(bool(transpose_a)), int(bool(transpose_b))
        p.activation = _cabi.ACTIVATIONS[activation if fuse_act else "linear"]
        p.bias_len = bias_len if fuse_bias else 0
        p.prelu_len = (prelu_len or 0) if fuse_act else 0
        p.leakyrelu_alpha = 0.2 if alpha is None else float(alpha)
        if activation == "gelu_erf":
            p.gelu_scale, p.gelu_half, p.gelu_one = [float(np.float32(v)) for v in gelu[:3]]
            p.gelu_divide = int(bool(gelu[3]))
        try:
            bias_id = dev(backend, bias) if fuse_bias and bias is not None else 0
            prelu_id = dev(backend, prelu) if fuse_act and activation == "prelu" else 0
            if heads is None:
                backend.check(backend.lib.tfjs_cuda_fused_matmul(
                    backend.ctx, byref(p), dev(backend, a), dev(backend, b), bias_id, prelu_id,
                    dev(backend, out)))
            else:
                backend.check(backend.lib.tfjs_cuda_fused_matmul_heads(
                    backend.ctx, byref(p), dev(backend, a), dev(backend, b), bias_id, prelu_id,
                    heads[0], heads[1], heads[2], dev(backend, out)))
        except Exception:
            backend.disposeData(out.dataId)
            raise
    if not fuse_bias:
        added = elementwise.binary_impl(backend, "Add", out, bias)
        backend.disposeData(out.dataId)
        out = added
    if not fuse_act:
        act = elementwise.apply_activation(backend, out, activation, prelu, alpha)
        backend.disposeData(out.dataId)
        out = act
    return out


def fused_matmul(args):
    i, a, b = args["inputs"], args["attrs"], args["backend"]
    return _matmul_impl(b, i["a"], i["b"], a.get("transposeA", False),
                        a.get("transposeB", False), i.get("bias"),
                        i.get("preluActivationWeights"), a.get("activation") or "linear",
                        a.get("leakyreluAlpha"), gelu=a.get("geluParams"))


def batch_matmul(args):
    i, a, b = args["inputs"], args["attrs"], args["backend"]
    return _matmul_impl(b, i["a"], i["b"], a.get("transposeA", False),
                        a.get("transposeB", False), None, None, "linear", None)


def matmul_heads(args):
    """The product of _FusedMatMul / BatchMatMul written through the permutation that splits
    or merges attention heads (what Reshape + Transpose([0, 2, 1, 3]) would do in a pass of
    its own).  attrs.layout "split": a [.., M, K] x b [K, N] with M = B*S, N = H*D gives
    [B, H, S, D]; "merge": a [B, H, S, K] x b [B, H, K, D] gives [B, S, H, D];
    attrs.heads = [B, S, H, D]."""
    i, at, backend = args["inputs"], args["attrs"], args["backend"]
    a, b = i["a"], i["b"]
    B, S, H, D = [int(v) for v in at["heads"]]
    ta, tb = at.get("transposeA", False), at.get("transposeB", False)
    m = a.shape[-1] if ta else a.shape[-2]
    n = b.shape[-2] if tb else b.shape[-1]
    batch = size_from_shape(a.shape[:-2])
    if at["layout"] == "split":
        ok = batch == 1 and size_from_shape(b.shape[:-2]) == 1 and m == B * S and n == H * D
        heads = (_cabi.HEADS_SPLIT, S, D, [B, H, S, D])
    else:
        ok = (list(a.shape[:-2]) == [B, H] and list(b.shape[:-2]) == [B, H] and m == S and n == D)
        heads = (_cabi.HEADS_MERGE, H, D, [B, S, H, D])
    if not ok:
        raise _cabi.CudaError(_cabi.UNSUPPORTED, "matMul heads: operand shapes %s %s do not "
                              "give heads %s" % (a.shape, b.shape, [B, S, H, D]))
    return _matmul_impl(backend, a, b, ta, tb, i.get("bias"), i.get("preluActivationWeights"),
                        at.get("activation") or "linear", at.get("leakyreluAlpha"), heads)


CONFIGS = [
    KernelConfig("_MatMulHeads", BACKEND, matmul_heads),
    KernelConfig("_FusedMatMul", BACKEND, fused_matmul),
    KernelConfig("BatchMatMul", BACKEND, batch_matmul),
]
