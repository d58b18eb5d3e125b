"""Convolution / pooling geometry, restated from tfjs-core/src/ops/conv_util.ts.

The kernels take explicit pads and output sizes; this module is where 'same' /
'valid' / numeric / explicit padding and the dimRoundingMode rules are turned
into numbers, exactly as computeConv2DInfo (conv_util.ts:177-236),
getPadAndOutInfo (:429-481) and computePool2DInfo (:119-140) do.
"""
import math


class Conv2DInfo(object):
    __slots__ = ("batchSize", "inHeight", "inWidth", "inChannels", "outHeight",
                 "outWidth", "outChannels", "dataFormat", "strideHeight",
                 "strideWidth", "dilationHeight", "dilationWidth", "filterHeight",
                 "filterWidth", "effectiveFilterHeight", "effectiveFilterWidth",
                 "padInfo", "inShape", "outShape", "filterShape")


def parse_tuple_param(param):
    """conv_util.ts:395-403."""
    if isinstance(param, (int, float)):
        return [int(param), int(param), int(param)]
    param = [int(p) for p in param]
    if len(param) == 2:
        return [param[0], param[1], 1]
    if len(param) == 1:
        return [param[0], param[0], param[0]]
    return param


def get_effective_filter_size(filter_size, dilation):
    """conv_util.ts:421-427."""
    if dilation <= 1:
        return filter_size
    return filter_size + (filter_size - 1) * (dilation - 1)


def _js_round(value):
    r = math.floor(value)
    return r + 1 if value - r >= 0.5 else r


def round_mode(value, rounding_mode=None):
    """conv_util.ts:548-564: no mode means truncation."""
    if not rounding_mode:
        return math.trunc(value)
    if rounding_mode == "round":
        return _js_round(value)
    if rounding_mode == "ceil":
        return math.ceil(value)
    if rounding_mode == "floor":
        return math.floor(value)
    raise ValueError("Unknown roundingMode %s" % rounding_mode)


def compute_output_shape_2d(in_shape, field_size, stride, zero_pad, rounding_mode):
    """conv_util.ts:350-365 (one field size and one stride for both axes)."""
    rows = round_mode((in_shape[0] - field_size + 2 * zero_pad) / stride + 1, rounding_mode)
    cols = round_mode((in_shape[1] - field_size + 2 * zero_pad) / stride + 1, rounding_mode)
    return rows, cols


def get_pad_and_out_info(pad, in_h, in_w, s_h, s_w, f_h, f_w, rounding_mode,
                         data_format="channelsLast"):
    """conv_util.ts:429-481."""
    if isinstance(pad, bool):
        raise ValueError("Unknown padding parameter: %r" % (pad,))
    if isinstance(pad, (int, float)):
        pad_type = "VALID" if pad == 0 else "NUMBER"
        info = dict(top=pad, bottom=pad, left=pad, right=pad, type=pad_type)
        out_h, out_w = compute_output_shape_2d([in_h, in_w], f_h, s_h, pad, rounding_mode)
    elif pad == "same":
        out_h = math.ceil(in_h / s_h)
        out_w = math.ceil(in_w / s_w)
        pad_h = max(0, (out_h - 1) * s_h + f_h - in_h)
        pad_w = max(0, (out_w - 1) * s_w + f_w - in_w)
        top = pad_h // 2
        left = pad_w // 2
        info = dict(top=top, bottom=pad_h - top, left=left, right=pad_w - left, type="SAME")
    elif pad == "valid":
        info = dict(top=0, bottom=0, left=0, right=0, type="VALID")
        out_h = math.ceil((in_h - f_h + 1) / s_h)
        out_w = math.ceil((in_w - f_w + 1) / s_w)
    elif isinstance(pad, (list, tuple)):
        hi, wi = (1, 2) if data_format == "channelsLast" else (2, 3)
        top, bottom = int(pad[hi][0]), int(pad[hi][1])
        left, right = int(pad[wi][0]), int(pad[wi][1])
        pad_type = "VALID" if top == bottom == left == right == 0 else "EXPLICIT"
        info = dict(top=top, bottom=bottom, left=left, right=right, type=pad_type)
        out_h = round_mode((in_h - f_h + top + bottom) / s_h + 1, rounding_mode)
        out_w = round_mode((in_w - f_w + left + right) / s_w + 1, rounding_mode)
    else:
        raise ValueError("Unknown padding parameter: %r" % (pad,))
    return info, out_h, out_w


def compute_conv2d_info(in_shape, filter_shape, strides, dilations, pad,
                        rounding_mode=None, depthwise=False,
                        data_format="channelsLast"):
    """conv_util.ts:177-236."""
    if data_format == "channelsLast":
        batch, in_h, in_w, in_c = [int(v) for v in in_shape]
    elif data_format == "channelsFirst":
        batch, in_c, in_h, in_w = [int(v) for v in in_shape]
    else:
        raise ValueError("Unknown dataFormat %s" % data_format)
    f_h, f_w, _, f_c = [int(v) for v in filter_shape]
    s_h, s_w = parse_tuple_param(strides)[:2]
    d_h, d_w = parse_tuple_param(dilations)[:2]
    eff_h = get_effective_filter_size(f_h, d_h)
    eff_w = get_effective_filter_size(f_w, d_w)
    pad_info, out_h, out_w = get_pad_and_out_info(pad, in_h, in_w, s_h, s_w, eff_h, eff_w,
                                                  rounding_mode, data_format)
    out_c = f_c * in_c if depthwise else f_c
    ci = Conv2DInfo()
    ci.batchSize, ci.inHeight, ci.inWidth, ci.inChannels = batch, in_h, in_w, in_c
    ci.outHeight, ci.outWidth, ci.outChannels = int(out_h), int(out_w), out_c
    ci.dataFormat = data_format
    ci.strideHeight, ci.strideWidth = s_h, s_w
    ci.dilationHeight, ci.dilationWidth = d_h, d_w
    ci.filterHeight, ci.filterWidth = f_h, f_w
    ci.effectiveFilterHeight, ci.effectiveFilterWidth = eff_h, eff_w
    ci.padInfo = pad_info
    ci.inShape = list(in_shape)
    ci.filterShape = list(filter_shape)
    if data_format == "channelsFirst":
        ci.outShape = [batch, out_c, ci.outHeight, ci.outWidth]
    else:
        ci.outShape = [batch, ci.outHeight, ci.outWidth, out_c]
    return ci


def compute_pool2d_info(in_shape, filter_size, strides, dilations, pad,
                        rounding_mode=None, data_format="channelsLast"):
    """conv_util.ts:119-140."""
    f_h, f_w = parse_tuple_param(filter_size)[:2]
    ch = in_shape[3] if data_format == "channelsLast" else in_shape[1]
    return compute_conv2d_info(in_shape, [f_h, f_w, ch, ch], strides, dilations, pad,
                               rounding_mode, False, data_format)


def check_pad_on_dim_rounding_mode(op_desc, pad, dim_rounding_mode):
    """conv_util.ts:600-625: dimRoundingMode requires integer numeric pads."""
    if dim_rounding_mode is None:
        return
    if isinstance(pad, str):
        raise ValueError("Error in %s: pad must be an integer when using "
                         "dimRoundingMode %s but got pad %s." % (op_desc, dim_rounding_mode, pad))
    if isinstance(pad, (int, float)):
        if int(pad) != pad:
            raise ValueError("Error in %s: pad must be an integer when using "
                             "dimRoundingMode %s but got pad %s." % (op_desc, dim_rounding_mode, pad))
    elif isinstance(pad, (list, tuple)):
        for p in pad:
            for v in p:
                if int(v) != v:
                    raise ValueError("Error in %s: pad must be an integer when using "
                                     "dimRoundingMode %s but got pad %s." %
                                     (op_desc, dim_rounding_mode, v))
    else:
        raise ValueError("Error in %s: Unknown padding parameter: %s" % (op_desc, pad))


def either_strides_or_dilations_are_one(strides, dilations):
    """conv_util.ts:571-574."""
    one = lambda p: all(v == 1 for v in parse_tuple_param(p))
    return one(strides) or one(dilations)
