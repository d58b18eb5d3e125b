"""Shape helpers restated from tfjs-core: util_base.ts, broadcast_util.ts,
axis_util.ts and segment_util.ts (only what the inference kernels use)."""


def size_from_shape(shape):
    n = 1
    for s in shape:
        n *= int(s)
    return n


def compute_strides(shape):
    """util_base.ts computeStrides, but with the full rank (last stride 1)."""
    strides = [1] * len(shape)
    for i in range(len(shape) - 2, -1, -1):
        strides[i] = strides[i + 1] * int(shape[i + 1])
    return strides


def assert_and_get_broadcast_shape(a, b):
    """tfjs-core/src/ops/broadcast_util.ts:65-100."""
    out = []
    n = max(len(a), len(b))
    for i in range(n):
        x = a[len(a) - i - 1] if i < len(a) else 1
        y = b[len(b) - i - 1] if i < len(b) else 1
        if x == 1:
            out.insert(0, y)
        elif y == 1:
            out.insert(0, x)
        elif x != y:
            raise ValueError("Operands could not be broadcast together with shapes "
                             "%s and %s." % (",".join(map(str, a)), ",".join(map(str, b))))
        else:
            out.insert(0, x)
    return [int(v) for v in out]


def parse_axis_param(axis, shape):
    """util_base.ts:600-632."""
    rank = len(shape)
    if axis is None:
        return list(range(rank))
    if isinstance(axis, (int, float)):
        axis = [axis]
    axis = [int(a) for a in axis]
    for a in axis:
        if not (-rank <= a < rank) and not (rank == 0 and a in (0, -1)):
            raise ValueError("All values in axis param must be in range [-%d, %d) but "
                             "got axis %s" % (rank, rank, axis))
    return [a + rank if a < 0 else a for a in axis]


def get_axes_permutation(axes, rank):
    """axis_util.ts:86-97: None when the axes already are the innermost ones."""
    if axes_are_inner_most_dims(axes, rank):
        return None
    result = [i for i in range(rank) if i not in axes]
    result.extend(axes)
    return result


def axes_are_inner_most_dims(axes, rank):
    """axis_util.ts:24-31."""
    for i in range(len(axes)):
        if axes[len(axes) - i - 1] != rank - 1 - i:
            return False
    return True


def get_inner_most_axes(num_axes, rank):
    """axis_util.ts:103-109."""
    return list(range(rank - num_axes, rank))


def compute_out_and_reduce_shapes(shape, axes):
    """axis_util.ts:49-63."""
    out_shape = [shape[d] for d in range(len(shape)) if d not in axes]
    reduce_shape = [shape[d] for d in axes]
    return out_shape, reduce_shape


def expand_shape_to_keep_dim(shape, axes):
    """axis_util.ts:65-69."""
    reduce_sub = [1] * len(axes)
    out, si, ri = [], 0, 0
    rank = len(shape) + len(axes)
    for d in range(rank):
        if d in axes:
            out.append(reduce_sub[ri]); ri += 1
        else:
            out.append(shape[si]); si += 1
    return out


def collect_gather_op_shape_info(x_shape, indices_shape, axis, batch_dims):
    """tfjs-core/src/ops/segment_util.ts:74-140."""
    indices_rank = len(indices_shape)
    x_rank = len(x_shape)
    if batch_dims != 0:
        if batch_dims < -indices_rank or batch_dims > indices_rank:
            raise ValueError("Expect batchDims in the range of [-%d, %d], but got %d" %
                             (indices_rank, indices_rank, batch_dims))
    if batch_dims < 0:
        batch_dims += indices_rank
    if batch_dims > x_rank:
        raise ValueError("batchDims (%d) must be less than rank(x) (%d)." % (batch_dims, x_rank))
    if axis < batch_dims:
        raise ValueError("batchDims (%d) must be less than or equal to axis (%d)." %
                         (batch_dims, axis))
    for i in range(batch_dims):
        if x_shape[i] != indices_shape[i]:
            raise ValueError("x.shape[%d]: %d should be equal to indices.shape[%d]: %d." %
                             (i, x_shape[i], i, indices_shape[i]))
    dim_size = x_shape[axis]
    output_shape = []
    batch_size = outer_size = slice_size = 1
    for i in range(batch_dims):
        output_shape.append(x_shape[i]); batch_size *= x_shape[i]
    for i in range(batch_dims, axis):
        output_shape.append(x_shape[i]); outer_size *= x_shape[i]
    for i in range(batch_dims, indices_rank):
        output_shape.append(indices_shape[i])
    for i in range(axis + 1, x_rank):
        output_shape.append(x_shape[i]); slice_size *= x_shape[i]
    return dict(batchSize=batch_size, sliceSize=slice_size, outerSize=outer_size,
                dimSize=dim_size, outputShape=output_shape)
