"""View-producing manipulation functions: permute_dims, broadcast_to, reshape,
expand_dims, squeeze, and the broadcast-shape rule.

Behaviour follows dpnp/tensor/_manipulation_functions.py:96-133 (broadcast
shape), :277-311 (broadcast_to: stride 0 for stretched extents), :525-559
(permute_dims) and dpnp/tensor/_reshape.py (reshape without a copy when the
strides allow it).
"""

from __future__ import annotations

import operator

import numpy as np

from ._usmarray import usm_ndarray


def normalize_axis_index(axis, ndim, argname="axis"):
    axis = operator.index(axis)
    if not (-ndim <= axis < ndim):
        raise np.exceptions.AxisError(axis, ndim, argname)
    return axis + ndim if axis < 0 else axis


def normalize_axis_tuple(axis, ndim, argname="axis"):
    if isinstance(axis, (int, np.integer)):
        axis = (axis,)
    axis = tuple(normalize_axis_index(a, ndim, argname) for a in axis)
    if len(set(axis)) != len(axis):
        raise ValueError(f"repeated axis in `{argname}` argument")
    return axis


def _broadcast_shape_impl(shapes):
    """Common shape of several shapes under NumPy broadcasting."""
    nd = max((len(s) for s in shapes), default=0)
    out = [1] * nd
    for s in shapes:
        pad = nd - len(s)
        for i, ext in enumerate(s):
            cur = out[pad + i]
            if cur == 1:
                out[pad + i] = ext
            elif ext != 1 and ext != cur:
                raise ValueError("operands could not be broadcast together with shapes " +
                                 " ".join(str(tuple(x)) for x in shapes))
    return tuple(out)


def broadcast_shapes(*shapes):
    return _broadcast_shape_impl([tuple(s) for s in shapes])


def permute_dims(x, axes):
    if not isinstance(x, usm_ndarray):
        raise TypeError(f"Expected usm_ndarray type, got {type(x)}.")
    axes = tuple(axes) if not isinstance(axes, (int, np.integer)) else (axes,)
    if len(axes) != x.ndim:
        raise ValueError("The length of the passed axes does not match to the number of usm_ndarray dimensions.")
    axes = normalize_axis_tuple(axes, x.ndim, "axes")
    return x._like(x._ptr, tuple(x.shape[a] for a in axes), tuple(x.strides[a] for a in axes))


def broadcast_to(x, shape):
    if not isinstance(x, usm_ndarray):
        raise TypeError(f"Expected usm_ndarray type, got {type(x)}.")
    if isinstance(shape, (int, np.integer)):
        shape = (shape,)
    shape = tuple(operator.index(s) for s in shape)
    if len(shape) < x.ndim:
        raise ValueError(f"Can not broadcast an array of shape {x.shape} to shape {shape}")
    pad = len(shape) - x.ndim
    strides = [0] * pad
    for ext_new, ext, st in zip(shape[pad:], x.shape, x.strides):
        if ext == ext_new:
            strides.append(st)
        elif ext == 1:
            strides.append(0)
        else:
            raise ValueError(f"Can not broadcast an array of shape {x.shape} to shape {shape}")
    return x._like(x._ptr, shape, strides)


def broadcast_arrays(*arrays):
    shape = _broadcast_shape_impl([a.shape for a in arrays])
    return [broadcast_to(a, shape) for a in arrays]


def expand_dims(x, axis):
    axes = normalize_axis_tuple(axis, x.ndim + (1 if isinstance(axis, (int, np.integer)) else len(axis)))
    shape, strides = list(x.shape), list(x.strides)
    for a in sorted(axes):
        shape.insert(a, 1)
        strides.insert(a, 0)
    return x._like(x._ptr, shape, strides)


def squeeze(x, axis=None):
    if axis is None:
        keep = [i for i, s in enumerate(x.shape) if s != 1]
    else:
        axes = normalize_axis_tuple(axis, x.ndim)
        for a in axes:
            if x.shape[a] != 1:
                raise ValueError("Cannot select an axis to squeeze out which has size not equal to one.")
        keep = [i for i in range(x.ndim) if i not in axes]
    return x._like(x._ptr, [x.shape[i] for i in keep], [x.strides[i] for i in keep])


def _reshape_strides(old_shape, old_strides, new_shape):
    """Strides that view the same elements in C order under `new_shape`, or None."""
    # group old dims into maximal chunks that are internally C-chained
    old = [(s, st) for s, st in zip(old_shape, old_strides) if s != 1]
    new_strides = [0] * len(new_shape)
    oi = 0
    ni = 0
    nnew = len(new_shape)
    while ni < nnew:
        if new_shape[ni] == 1:
            new_strides[ni] = 1
            ni += 1
            continue
        if oi >= len(old):
            return None
        # grow a chunk of old dims and a chunk of new dims until their sizes agree
        o_size, o_first, o_last = old[oi][0], oi, oi
        n_size, n_first = new_shape[ni], ni
        nj = ni
        while o_size != n_size:
            if o_size < n_size:
                o_last += 1
                if o_last >= len(old):
                    return None
                if old[o_last - 1][1] != old[o_last][0] * old[o_last][1]:
                    return None
                o_size *= old[o_last][0]
            else:
                nj += 1
                while nj < nnew and new_shape[nj] == 1:
                    new_strides[nj] = 1
                    nj += 1
                if nj >= nnew:
                    return None
                n_size *= new_shape[nj]
        # strides inside the new chunk, innermost first
        st = old[o_last][1]
        for k in range(nj, n_first - 1, -1):
            if new_shape[k] == 1:
                new_strides[k] = 1
                continue
            new_strides[k] = st
            st *= new_shape[k]
        oi = o_last + 1
        ni = nj + 1
    if oi != len(old):
        return None
    return tuple(new_strides)


def reshape(x, shape, /, *, order="C", copy=None):
    if not isinstance(x, usm_ndarray):
        raise TypeError(f"Expected usm_ndarray type, got {type(x)}.")
    if order not in ("C", "c", "F", "f"):
        raise ValueError(f"Keyword 'order' not recognized. Expecting 'C' or 'F', got {order}")
    if isinstance(shape, (int, np.integer)):
        shape = (shape,)
    shape = [operator.index(s) for s in shape]
    neg = [i for i, s in enumerate(shape) if s < 0]
    if len(neg) > 1 or any(s < -1 for s in shape):
        raise ValueError("Only one dimension can have -1 as its extent")
    size = x.size
    if neg:
        known = 1
        for i, s in enumerate(shape):
            if i != neg[0]:
                known *= s
        if known == 0 or size % known:
            raise ValueError(f"Can not reshape array of size {size} into {tuple(shape)}")
        shape[neg[0]] = size // known
    n = 1
    for s in shape:
        n *= s
    if n != size:
        raise ValueError(f"Can not reshape array of size {size} into {tuple(shape)}")
    shape = tuple(shape)
    if order in ("F", "f"):
        r = reshape(x.T, shape[::-1], copy=copy)
        return r.T
    if size == 0:
        from ._usmarray import _dense_strides
        return x._like(x._ptr, shape, _dense_strides(shape))
    new_strides = None if copy is True else _reshape_strides(x.shape, x.strides, shape)
    if new_strides is not None:
        return x._like(x._ptr, shape, new_strides)
    if copy is False:
        raise ValueError("Reshaping the array requires a copy, but no copying was requested by using copy=False")
    from ._copy_utils import copy as _copy
    c = _copy(x, order="C")
    from ._usmarray import _dense_strides
    return c._like(c._ptr, shape, _dense_strides(shape))


def flip(x, /, *, axis=None):
    """Reverse the order of elements along the given axes (a view with negated strides)."""
    if not isinstance(x, usm_ndarray):
        raise TypeError(f"Expected usm_ndarray type, got {type(x)}.")
    axes = tuple(range(x.ndim)) if axis is None else normalize_axis_tuple(axis, x.ndim)
    key = tuple(slice(None, None, -1) if i in axes else slice(None) for i in range(x.ndim))
    return x[key]
