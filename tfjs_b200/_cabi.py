"""ctypes binding of libtfjs_cuda.so (the C ABI declared in include/tfjs_cuda.h).

This is the Python stand-in for the N-API addon: it forwards calls one to one
and turns non-zero status codes into exceptions, the way the TypeScript side
turns them into `throw new Error(msg)`.  There is no fallback: if the shared
library is missing, importing a backend fails loudly.
"""
import ctypes
import os
from ctypes import (POINTER, Structure, byref, c_char_p, c_double, c_float,
                    c_int, c_int32, c_int64, c_uint32, c_uint64, c_void_p)

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libtfjs_cuda.so")

OK = 0
UNSUPPORTED = 5
ACTIVATIONS = dict(linear=0, relu=1, relu6=2, prelu=3, leakyrelu=4, sigmoid=5,
                   elu=6, gelu_erf=7)
DTYPES = dict(float32=0, int32=1, bool=2)
BINARY_OPS = dict(Add=0, Sub=1, Multiply=2, RealDiv=3, Maximum=4, Minimum=5,
                  Pow=6, SquaredDifference=7, Prelu=8)
UNARY_OPS = dict(Relu=0, Relu6=1, Elu=2, Sigmoid=3, LeakyRelu=4, Exp=5, Sqrt=6,
                 Rsqrt=7, Square=8, Tanh=9, Neg=10, ClipByValue=11, Erf=12,
                 Abs=13, Log=14)
REDUCE_OPS = dict(Sum=0, Mean=1, Max=2)
MATH_TF32, MATH_FP32 = 0, 1


class Conv2DParams(Structure):
    _fields_ = [(n, c_int32) for n in (
        "batch", "in_h", "in_w", "in_c", "out_h", "out_w", "out_c", "filter_h",
        "filter_w", "stride_h", "stride_w", "dilation_h", "dilation_w",
        "pad_top", "pad_left", "activation", "bias_len", "prelu_len")] + [
            ("leakyrelu_alpha", c_double)]


EW_MAX_INPUTS, EW_MAX_OPS, EW_UNARY = 8, 24, 32
EW_FULL, EW_PERIODIC, EW_ROW, EW_SCALAR, EW_BATCHED = 0, 1, 2, 3, 4


class EwOp(Structure):
    _fields_ = [("opcode", ctypes.c_int16), ("a", ctypes.c_uint8), ("b", ctypes.c_uint8),
                ("p0", c_float), ("p1", c_float)]


class EwProgram(Structure):
    _fields_ = [("n_inputs", c_int32), ("n_ops", c_int32), ("n", c_uint64),
                ("cols", c_uint32), ("reserved", c_uint32),
                ("input_id", c_int32 * EW_MAX_INPUTS), ("input_mode", c_int32 * EW_MAX_INPUTS),
                ("input_period", c_uint32 * EW_MAX_INPUTS),
                ("input_aux", c_uint32 * EW_MAX_INPUTS), ("ops", EwOp * EW_MAX_OPS)]


class MatMulParams(Structure):
    _fields_ = [(n, c_int32) for n in (
        "batch_a", "batch_b", "m", "n", "k", "transpose_a", "transpose_b",
        "activation", "bias_len", "prelu_len")] + [
            ("leakyrelu_alpha", c_double), ("gelu_scale", c_float), ("gelu_half", c_float),
            ("gelu_one", c_float), ("gelu_divide", c_int32)]


STORED_RAW, STORED_UINT8, STORED_UINT16, STORED_FLOAT16 = 0, 1, 2, 3


class WeightSpec(Structure):
    _fields_ = [("n", c_uint64), ("storage", c_int32), ("dtype", c_int32), ("scale", c_double),
                ("min", c_double), ("skip", c_int32), ("reserved", c_int32)]


# name -> (restype, argtypes); every symbol include/tfjs_cuda.h declares.
_CTX = c_void_p
_I64P = POINTER(c_int64)
SIGNATURES = {
    "tfjs_cuda_device_count": (c_int, [POINTER(c_int)]),
    "tfjs_cuda_create": (c_int, [c_int, POINTER(_CTX)]),
    "tfjs_cuda_destroy": (None, [_CTX]),
    "tfjs_cuda_last_error": (c_char_p, [_CTX]),
    "tfjs_cuda_alloc": (c_int, [_CTX, c_uint64, POINTER(c_int32)]),
    "tfjs_cuda_free": (c_int, [_CTX, c_int32]),
    "tfjs_cuda_write": (c_int, [_CTX, c_int32, c_void_p, c_uint64]),
    "tfjs_cuda_upload": (c_int, [_CTX, c_void_p, c_uint64, POINTER(c_int32)]),
    "tfjs_cuda_read": (c_int, [_CTX, c_int32, c_void_p, c_uint64]),
    "tfjs_cuda_read_async": (c_int, [_CTX, c_int32, c_void_p, c_uint64]),
    "tfjs_cuda_sync": (c_int, [_CTX]),
    "tfjs_cuda_size_of": (c_int, [_CTX, c_int32, POINTER(c_uint64)]),
    "tfjs_cuda_device_ptr": (c_int, [_CTX, c_int32, POINTER(c_void_p)]),
    "tfjs_cuda_memory": (c_int, [_CTX] + [POINTER(c_uint64)] * 4),
    "tfjs_cuda_trim": (c_int, [_CTX]),
    "tfjs_cuda_host_alloc": (c_int, [_CTX, c_uint64, POINTER(c_void_p)]),
    "tfjs_cuda_host_free": (c_int, [_CTX, c_void_p]),
    "tfjs_cuda_time_begin": (c_int, [_CTX]),
    "tfjs_cuda_time_end": (c_int, [_CTX, POINTER(c_float)]),
    "tfjs_cuda_event_record": (c_int, [_CTX, c_int32]),
    "tfjs_cuda_event_elapsed": (c_int, [_CTX, c_int32, c_int32, POINTER(c_float)]),
    "tfjs_cuda_set_math_mode": (c_int, [_CTX, c_int]),
    "tfjs_cuda_launch_count": (c_int, [_CTX, POINTER(c_uint64)]),
    "tfjs_cuda_flush_l2": (c_int, [_CTX]),
    "tfjs_cuda_launch_log": (c_int, [_CTX, c_int32]),
    "tfjs_cuda_launch_log_take": (c_int, [_CTX, c_char_p, c_uint64, POINTER(c_uint32)]),
    "tfjs_cuda_fused_conv2d": (c_int, [_CTX, POINTER(Conv2DParams)] + [c_int32] * 5),
    "tfjs_cuda_fused_elementwise": (c_int, [_CTX, POINTER(EwProgram), c_int32]),
    "tfjs_cuda_fused_elementwise_catalogued": (c_int, [_CTX, POINTER(EwProgram),
                                                       POINTER(c_int32)]),
    "tfjs_cuda_decode_float16": (c_int, [_CTX, c_int32, c_uint64, c_int32]),
    "tfjs_cuda_capture_begin": (c_int, [_CTX, c_uint64]),
    "tfjs_cuda_capture_end": (c_int, [_CTX, c_int, POINTER(c_int32)]),
    "tfjs_cuda_graph_launch": (c_int, [_CTX, c_int32]),
    "tfjs_cuda_graph_destroy": (c_int, [_CTX, c_int32]),
    "tfjs_cuda_copy": (c_int, [_CTX, c_int32, c_int32, c_uint64]),
    "tfjs_cuda_high_water_reset": (c_int, [_CTX]),
    "tfjs_cuda_read_begin": (c_int, [_CTX, c_int32, c_void_p, c_uint64, POINTER(c_int32)]),
    "tfjs_cuda_read_wait": (c_int, [_CTX, c_int32]),
    "tfjs_cuda_fused_conv2d_residual": (c_int, [_CTX, POINTER(Conv2DParams)] + [c_int32] * 7),
    "tfjs_cuda_fused_depthwise_project": (c_int, [_CTX, POINTER(Conv2DParams), POINTER(Conv2DParams)]
                                          + [c_int32] * 8),
    "tfjs_cuda_add_activation": (c_int, [_CTX, c_int32, c_int32, c_int32, c_uint64, c_int32]),
    "tfjs_cuda_fused_depthwise_conv2d": (c_int, [_CTX, POINTER(Conv2DParams)] + [c_int32] * 5),
    "tfjs_cuda_fused_matmul": (c_int, [_CTX, POINTER(MatMulParams)] + [c_int32] * 5),
    "tfjs_cuda_fused_matmul_heads": (c_int, [_CTX, POINTER(MatMulParams)] + [c_int32] * 8),
    "tfjs_cuda_fused_matmul_group": (c_int, [_CTX, POINTER(MatMulParams), c_int32, c_int32,
                                     POINTER(c_int32), POINTER(c_int32), c_int32, c_int32,
                                     c_int32, POINTER(c_int32)]),
    "tfjs_cuda_pool2d": (c_int, [_CTX, POINTER(Conv2DParams), c_int32, c_int32, c_int32]),
    "tfjs_cuda_binary": (c_int, [_CTX, c_int32, c_int32, c_int32, c_int32, _I64P,
                                 c_int32, _I64P, c_int32, _I64P]),
    "tfjs_cuda_unary": (c_int, [_CTX, c_int32, c_double, c_double, c_int32,
                                c_uint64, c_int32]),
    "tfjs_cuda_softmax": (c_int, [_CTX, c_int32, c_uint64, c_uint64, c_int32]),
    "tfjs_cuda_softmax_scaled_masked": (c_int, [_CTX, c_int32, c_uint64, c_uint64, c_int32, c_float,
                                                c_int32, c_uint64, c_int32]),
    "tfjs_cuda_fused_attention": (c_int, [_CTX, c_int32, c_int32, c_int32, c_int32, c_int32,
                                          c_float, c_int32, c_int32, c_int32, c_int32, c_int32,
                                          c_int32]),
    "tfjs_cuda_layer_norm": (c_int, [_CTX, c_int32, c_int32, c_int32, c_int32, c_uint64, c_uint64,
                                     c_float, c_int32]),
    "tfjs_cuda_reduce": (c_int, [_CTX, c_int32, c_int32, c_uint64, c_uint64,
                                 c_uint64, c_int32]),
    "tfjs_cuda_argmax": (c_int, [_CTX, c_int32, c_uint64, c_uint64, c_uint64,
                                 c_int32]),
    "tfjs_cuda_transpose": (c_int, [_CTX, c_int32, c_int32, c_int32, _I64P,
                                    POINTER(c_int32), c_int32]),
    "tfjs_cuda_gather": (c_int, [_CTX, c_int32, c_int32, c_int32, c_uint64,
                                 c_uint64, c_uint64, c_uint64, c_uint64, c_int32,
                                 c_int32, _I64P]),
    "tfjs_cuda_cast": (c_int, [_CTX, c_int32, c_int32, c_int32, c_uint64, c_int32]),
    "tfjs_cuda_copy_strided": (c_int, [_CTX, c_int32, c_int32, _I64P, c_int32,
                                       c_int64, _I64P, _I64P, c_int32, c_int64,
                                       _I64P]),
    "tfjs_cuda_fill": (c_int, [_CTX, c_int32, c_uint32, c_int32, c_uint64]),
    "tfjs_cuda_batchnorm": (c_int, [_CTX, c_int32, c_uint64, c_int32, c_uint64,
                                    c_int32, c_uint64, c_int32, c_uint64, c_int32,
                                    c_uint64, c_double, c_int32]),
    "tfjs_cuda_batchnorm_rows": (c_int, [_CTX, c_int32, c_uint64, c_uint64] + [c_int32] * 8 +
                                 [c_double, c_int32]),
    "tfjs_cuda_dequantize": (c_int, [_CTX, c_int32, c_int32, c_int32, c_double,
                                     c_double, c_uint64, c_int32]),
    "tfjs_cuda_weights_begin": (c_int, [_CTX, POINTER(WeightSpec), c_int32, POINTER(c_int32)]),
    "tfjs_cuda_weights_push": (c_int, [_CTX, c_int32, c_void_p, c_uint64]),
    "tfjs_cuda_weights_push_file": (c_int, [_CTX, c_int32, c_char_p]),
    "tfjs_cuda_weights_end": (c_int, [_CTX, c_int32, POINTER(c_int32), POINTER(c_uint64)]),
    "tfjs_cuda_dequantize_static": (c_int, [_CTX, c_int32, c_int32, c_int32, c_double,
                                            c_double, c_uint64, c_int32]),
}

_lib = None


def load():
    """Load the shared library; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            "libtfjs_cuda.so is missing (%s). Build it with "
            "`make -C tfjs_b200/csrc`; this backend has no CPU fallback." % LIB_PATH)
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if a declared symbol is absent
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


HEADS_SPLIT, HEADS_MERGE = 1, 2


class CudaError(RuntimeError):
    def __init__(self, code, message):
        super().__init__(message)
        self.code = code


def i64(values):
    return (c_int64 * max(len(values), 1))(*[int(v) for v in values])


def i32(values):
    return (c_int32 * max(len(values), 1))(*[int(v) for v in values])
