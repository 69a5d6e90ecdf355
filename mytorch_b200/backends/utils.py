"""Shape arithmetic shared by the operator wrappers (broadcast, reduce and reshape rules of
``mytorch/backends/utils.py:6-70``)."""
import math


def calculate_broadcast_shape(x_shape, y_shape):
    nd = max(len(x_shape), len(y_shape))
    xs = (1,) * (nd - len(x_shape)) + tuple(x_shape)
    ys = (1,) * (nd - len(y_shape)) + tuple(y_shape)
    out = []
    for a, b in zip(xs, ys):
        if a != b and a != 1 and b != 1:
            raise RuntimeError(f"Invalid broadcast shape: {tuple(x_shape)} and {tuple(y_shape)}")
        out.append(max(a, b))
    return tuple(out)


def calculate_reduce_shape(shape, dim, keepdim):
    for i in dim:
        if not isinstance(i, int) or not 0 <= i < len(shape):
            raise RuntimeError(f"Reduce dim is invalid: {dim}")
    if keepdim:
        return tuple(1 if i in dim else s for i, s in enumerate(shape))
    return tuple(s for i, s in enumerate(shape) if i not in dim)


def calculate_reshaped_shape(original_shape, target_shape):
    total = math.prod(original_shape)
    target_shape = tuple(target_shape)
    known, unknown = 1, None
    for i, d in enumerate(target_shape):
        if d == -1:
            if unknown is not None:
                raise ValueError("can only specify one unknown dimension")
            unknown = i
        elif d <= 0:
            raise ValueError("negative dimensions not allowed except -1")
        else:
            known *= d
    if unknown is None:
        if known != total:
            raise ValueError(f"cannot reshape array of size {total} into shape {target_shape}")
        return target_shape
    if total % known != 0:
        raise ValueError(f"cannot reshape array of size {total} into shape {target_shape}")
    return target_shape[:unknown] + (total // known,) + target_shape[unknown + 1:]
