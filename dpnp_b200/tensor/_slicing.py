"""Basic (view-producing) indexing.

Restates ``_basic_slice_meta`` of the reference (dpnp/tensor/_slicing.pyx:128-...):
integers drop a dimension, slices scale the stride and move the offset,
``None`` inserts an extent-1 dimension, an ellipsis expands to full slices.
"""

from __future__ import annotations

import operator


def basic_slice_meta(key, shape, strides):
    """Return (new_shape, new_strides, element_offset, has_advanced_index)."""
    if not isinstance(key, tuple):
        key = (key,)
    n_explicit = 0
    ellipsis_seen = False
    for k in key:
        if k is Ellipsis:
            if ellipsis_seen:
                raise IndexError("an index can only have a single ellipsis ('...')")
            ellipsis_seen = True
        elif k is None:
            pass
        elif isinstance(k, slice):
            n_explicit += 1
        elif hasattr(k, "__index__") and not hasattr(k, "shape"):
            n_explicit += 1
        elif hasattr(k, "shape") and getattr(k, "ndim", 1) == 0 and getattr(k, "dtype", None) is not None \
                and k.dtype.kind in "iu":
            n_explicit += 1
        else:
            return None, None, 0, True
    nd = len(shape)
    if n_explicit > nd:
        raise IndexError(f"too many indices for an array of {nd} dimensions")
    new_shape, new_strides = [], []
    offset = 0
    dim = 0
    for k in key:
        if k is Ellipsis:
            fill = nd - n_explicit
            for _ in range(fill):
                new_shape.append(shape[dim])
                new_strides.append(strides[dim])
                dim += 1
        elif k is None:
            new_shape.append(1)
            new_strides.append(0)
        elif isinstance(k, slice):
            start, stop, step = k.indices(shape[dim])
            if step > 0:
                length = max(0, (stop - start + step - 1) // step)
            else:
                length = max(0, (start - stop - step - 1) // (-step))
            new_shape.append(length)
            new_strides.append(strides[dim] * step)
            if length > 0:
                offset += start * strides[dim]
            dim += 1
        else:
            i = operator.index(k)
            if not (-shape[dim] <= i < shape[dim]):
                raise IndexError(f"Index {i} is out of range for axes {dim} with size {shape[dim]}")
            if i < 0:
                i += shape[dim]
            offset += i * strides[dim]
            dim += 1
    while dim < nd:
        new_shape.append(shape[dim])
        new_strides.append(strides[dim])
        dim += 1
    # an empty result keeps pointing inside the allocation
    n = 1
    for s in new_shape:
        n *= s
    if n == 0:
        offset = 0
    return tuple(new_shape), tuple(new_strides), offset, False
