"""Arrays sharded along their leading axis over the GPUs of one box, one process per GPU.

:class:`ShardedArray` lets the unchanged API work on an array that is too large for, or simply
spread over, several GPUs: every rank holds the rows ``shard_bounds(n, world, rank)`` of the
whole array and calls the same functions --

    x = sharded.from_local(my_rows, comm)          # or sharded.scatter_rows(...)
    y = dp.exp(x) * 2.0 + x                        # slabs: no communication
    dp.sum(x, axis=1)                              # rows stay whole: no communication
    dp.sum(x, axis=0), dp.mean(x), dp.max(x)       # one partial per rank + one combine
    dp.argmax(x)                                   # first occurrence across shards

Elementwise functions of identically sharded operands (and of a sharded operand with scalars or
with plain arrays that broadcast along the non-sharded axes) give sharded results.  A reduction
that keeps the leading axis gives a sharded result; one that removes it combines the ranks'
partials and gives every rank the same plain array:

* sums: all-gather of the partials and one kernel that adds them in rank order -- the same bits on
  every rank, independent of the order in which the collective moves data;
* max / min: the same with the NaN-propagating maximum / minimum;
* argmax / argmin over everything: (value, global index) records, all-gathered, winner picked on
  the device: better value, ties to the smaller index, NaN is extreme.

Operands sharded differently, or living in different groups, raise ``ExecutionPlacementError``
as arrays on different queues do in the reference's compute-follows-data rule
(dpnp/tensor/_compute_follows_data.pyx:67-160, dpnp/tensor/_elementwise_common.py:240-254); the
reference itself has no multi-device arrays, so everything else here is new functionality.

The combines take device arrays (NCCL through the C ABI, :mod:`dpnp_b200._comm`) or NumPy arrays
(host messages); shards held as NumPy arrays exist so that the sharding rules can be tested on a
machine without a GPU -- the library never computes device arrays' results on the host.
"""

from __future__ import annotations

import numpy as np

from ._comm import Communicator, HostGroup
from .memory import ExecutionPlacementError

__all__ = ["ShardedArray", "shard_bounds", "init", "from_local", "scatter_rows", "Communicator", "HostGroup"]

_default_comm = [None]


def shard_bounds(n: int, world_size: int, rank: int) -> tuple[int, int]:
    """Half-open range of leading-axis indices owned by `rank` (sizes differ by at most one)."""
    base, extra = divmod(int(n), int(world_size))
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def init(comm: Communicator | None = None) -> Communicator:
    """The job's communicator (made from the launcher's environment on first use)."""
    if comm is not None:
        _default_comm[0] = comm
    elif _default_comm[0] is None:
        _default_comm[0] = Communicator()
    return _default_comm[0]


def _xp(local):
    """Array namespace of a shard: this library for device arrays, NumPy for host arrays."""
    if isinstance(local, np.ndarray):
        return np
    import dpnp_b200

    return dpnp_b200


def from_local(local, comm: Communicator | None = None, global_rows: int | None = None) -> "ShardedArray":
    """Sharded array whose part on this rank is `local` (rows `shard_bounds(...)` of the whole)."""
    comm = init(comm)
    counts = comm.host.allgather_object((int(local.shape[0]), tuple(local.shape[1:]), str(local.dtype)))
    if any(c[1:] != counts[0][1:] for c in counts):
        raise ValueError(f"shards disagree in trailing shape or type: {counts}")
    rows = [c[0] for c in counts]
    total = sum(rows)
    if global_rows is not None and global_rows != total:
        raise ValueError(f"shards hold {total} rows, expected {global_rows}")
    for r, n in enumerate(rows):
        lo, hi = shard_bounds(total, comm.world, r)
        if n != hi - lo:
            raise ValueError(f"rank {r} holds {n} rows; an even split of {total} rows gives it {hi - lo}")
    return ShardedArray(local, (total,) + tuple(local.shape[1:]), comm)


def scatter_rows(global_array, comm: Communicator | None = None) -> "ShardedArray":
    """Sharded array from a host array every rank holds whole: each rank keeps (and, with a GPU,
    uploads) its own rows."""
    comm = init(comm)
    a = np.asarray(global_array)
    if a.ndim == 0:
        raise ValueError("a 0-d array has no leading axis to shard")
    lo, hi = shard_bounds(a.shape[0], comm.world, comm.rank)
    mine = np.ascontiguousarray(a[lo:hi])
    if comm.queue is not None:
        import dpnp_b200 as dp

        mine = dp.asarray(mine, sycl_queue=comm.queue)
    return ShardedArray(mine, a.shape, comm)


def _identity_for(dtype, op):
    dtype = np.dtype(dtype)
    if dtype.kind == "f":
        return -np.inf if op == "max" else np.inf
    if dtype.kind == "b":
        return op != "max"
    info = np.iinfo(dtype)
    return info.min if op == "max" else info.max


class ShardedArray:
    """Rows ``shard_bounds(shape[0], world, rank)`` of an array of `shape`, one part per rank."""

    __array_priority__ = 300.0
    __array_ufunc__ = None

    def __init__(self, local, global_shape, comm: Communicator):
        global_shape = tuple(int(s) for s in global_shape)
        if len(global_shape) == 0 or len(global_shape) != local.ndim:
            raise ValueError("the whole array must have the shard's number of dimensions (at least 1)")
        lo, hi = shard_bounds(global_shape[0], comm.world, comm.rank)
        if tuple(local.shape) != (hi - lo,) + global_shape[1:]:
            raise ValueError(f"rank {comm.rank} of {comm.world} must hold a shard of shape "
                             f"{(hi - lo,) + global_shape[1:]}, got {tuple(local.shape)}")
        self.local = local
        self.shape = global_shape
        self.comm = comm
        self.row_offset = lo

    # ------------------------------------------------------------ attributes
    dtype = property(lambda self: self.local.dtype)
    ndim = property(lambda self: len(self.shape))
    size = property(lambda self: int(np.prod(self.shape, dtype=np.int64)))

    def __repr__(self):
        return (f"<ShardedArray {self.shape} {self.dtype}: rank {self.comm.rank}/{self.comm.world} holds rows "
                f"{self.row_offset}:{self.row_offset + self.local.shape[0]}>")

    def _new(self, local):
        return ShardedArray(local, (self.shape[0],) + tuple(local.shape[1:]), self.comm)

    def gather(self):
        """The whole array on every rank (a plain array of the shards' kind)."""
        xp = _xp(self.local)
        loc = self.local if isinstance(self.local, np.ndarray) else xp.ascontiguousarray(self.local)
        counts = [shard_bounds(self.shape[0], self.comm.world, r) for r in range(self.comm.world)]
        return self.comm.allgather(loc, [hi - lo for lo, hi in counts])

    def asnumpy(self):
        g = self.gather()
        return g if isinstance(g, np.ndarray) else g.asnumpy()

    # --------------------------------------------------------- elementwise
    def _operand(self, other):
        """`other` as the operand of a slab-wise operation with self, or an error."""
        if isinstance(other, ShardedArray):
            if other.comm is not self.comm:
                raise ExecutionPlacementError("sharded operands belong to different process groups")
            if other.shape[0] != self.shape[0] or other.ndim != self.ndim:
                raise ExecutionPlacementError(
                    f"operands are sharded differently: {self.shape} and {other.shape} "
                    "(elementwise functions need the same number of rows and dimensions)")
            return other.local
        if isinstance(other, (bool, int, float, complex, np.generic)):
            return other
        shape = getattr(other, "shape", None)
        if shape is None:
            raise TypeError(f"unsupported operand of type {type(other)}")
        # a plain array is the same on every rank: it may only broadcast along the sharded axis
        if len(shape) > self.ndim or (len(shape) == self.ndim and shape[0] != 1):
            raise ExecutionPlacementError(
                f"a plain array of shape {tuple(shape)} spans the sharded axis of {self.shape}; "
                "shard it the same way first")
        return other

    def _elementwise(self, name, *others, reflected=False, **kwargs):
        xp = _xp(self.local)
        args = [self._operand(o) for o in others]
        fn = getattr(xp, name)
        ops = ([*args, self.local] if reflected else [self.local, *args])
        out = kwargs.get("out")
        if out is not None:
            if not isinstance(out, ShardedArray):
                raise TypeError("out= of a sharded operation must be a sharded array")
            kwargs["out"] = self._operand(out)
            fn(*ops, **kwargs)
            return out
        return self._new(fn(*ops, **kwargs))

    def __add__(self, o): return self._elementwise("add", o)
    def __radd__(self, o): return self._elementwise("add", o, reflected=True)
    def __sub__(self, o): return self._elementwise("subtract", o)
    def __rsub__(self, o): return self._elementwise("subtract", o, reflected=True)
    def __mul__(self, o): return self._elementwise("multiply", o)
    def __rmul__(self, o): return self._elementwise("multiply", o, reflected=True)
    def __truediv__(self, o): return self._elementwise("divide", o)
    def __rtruediv__(self, o): return self._elementwise("divide", o, reflected=True)
    def __pow__(self, o): return self._elementwise("power", o)
    def __neg__(self): return self._elementwise("negative")
    def __abs__(self): return self._elementwise("abs")
    def __lt__(self, o): return self._elementwise("less", o)
    def __le__(self, o): return self._elementwise("less_equal", o)
    def __gt__(self, o): return self._elementwise("greater", o)
    def __ge__(self, o): return self._elementwise("greater_equal", o)
    def __eq__(self, o): return self._elementwise("equal", o)
    def __ne__(self, o): return self._elementwise("not_equal", o)
    __hash__ = None

    # ----------------------------------------------------------- reductions
    def _axes(self, axis):
        if axis is None:
            return tuple(range(self.ndim))
        axes = axis if isinstance(axis, (tuple, list)) else (axis,)
        out = []
        for a in axes:
            a = int(a)
            if not -self.ndim <= a < self.ndim:
                raise np.exceptions.AxisError(a, self.ndim)
            a %= self.ndim
            if a in out:
                raise ValueError("repeated axis")
            out.append(a)
        return tuple(out)

    def _keep(self, res, axes, keepdims):
        """Shape of a combined (replicated) result."""
        if not keepdims:
            return res
        shape = tuple(1 if i in axes else s for i, s in enumerate(self.shape))
        return res.reshape(shape)

    def _reduce(self, op, axis=None, dtype=None, keepdims=False, out=None):
        """sum / prod are not both here on purpose: only sum, max, min combine across ranks."""
        xp = _xp(self.local)
        axes = self._axes(axis)
        if out is not None:
            raise NotImplementedError("out= is not supported for reductions of sharded arrays")
        kw = {} if dtype is None else {"dtype": dtype}
        if 0 not in axes:
            # whole lanes live on one rank: nothing to exchange, the result stays sharded
            return self._new(getattr(xp, op)(self.local, axis=axes, keepdims=keepdims, **kw))
        if op == "sum":
            part = xp.sum(self.local, axis=axes, **kw)
            return self._keep(self.comm.sum_ordered(part), axes, keepdims)
        if op in ("max", "min"):
            if self.size == 0:
                raise ValueError("reduction cannot be performed over zero-size axes")
            if self.local.shape[0] == 0:
                # this rank owns no rows: it contributes the operation's identity
                shape = tuple(s for i, s in enumerate(self.shape) if i not in axes)
                part = xp.full(shape, _identity_for(self.dtype, op), dtype=self.dtype)
            else:
                part = getattr(xp, op)(self.local, axis=axes)
            return self._keep(self.comm.extreme(part, op), axes, keepdims)
        raise NotImplementedError(f"{op} over the sharded axis")

    def _mean(self, axis=None, keepdims=False):
        xp = _xp(self.local)
        axes = self._axes(axis)
        if 0 not in axes:
            return self._new(xp.mean(self.local, axis=axes, keepdims=keepdims))
        res_dt = self.dtype if np.dtype(self.dtype).kind in "fc" else np.dtype("f8")
        count = 1
        for a in axes:
            count *= self.shape[a]
        total = self.comm.sum_ordered(xp.sum(self.local, axis=axes, dtype=res_dt))
        # one division of the combined sum, as the single-device mean does after its sum
        return self._keep(total / res_dt.type(count) if isinstance(total, np.ndarray) else xp.divide(total, float(count)),
                          axes, keepdims)

    def _arg(self, op, axis=None, keepdims=False):
        xp = _xp(self.local)
        name = "argmax" if op == "max" else "argmin"
        if axis is not None:
            if isinstance(axis, (tuple, list)):
                raise TypeError("'axis' argument expected to have type 'int' or be `None`")
            axes = self._axes(axis)
            if axes != (0,):
                return self._new(getattr(xp, name)(self.local, axis=axes[0], keepdims=keepdims))
            return self._arg_leading(op, keepdims)
        if self.size == 0:
            raise ValueError("reduction cannot be performed over zero-size axes")
        per_row = 1
        for s in self.shape[1:]:
            per_row *= s
        loc = self.local if isinstance(self.local, np.ndarray) else xp.ascontiguousarray(self.local)
        li = getattr(xp, name)(loc) if loc.shape[0] else None
        _, idx = self.comm.arg_extreme(loc, li, self.row_offset * per_row, op)
        if keepdims:
            idx = idx.reshape((1,) * self.ndim)
        return idx

    def _arg_leading(self, op, keepdims):
        """argmax / argmin along the sharded axis: the global extreme per lane, then the smallest
        row among the ranks that reach it (two small combines)."""
        xp = _xp(self.local)
        name = "argmax" if op == "max" else "argmin"
        if self.shape[0] == 0:
            raise ValueError("reduction cannot be performed over zero-size axes")
        lane_shape = self.shape[1:]
        big = np.iinfo(np.int64).max
        if self.local.shape[0] == 0:
            vals = xp.full(lane_shape, _identity_for(self.dtype, op), dtype=self.dtype)
            rows = xp.full(lane_shape, big, dtype="i8")
        else:
            vals = getattr(xp, op)(self.local, axis=0)
            rows = getattr(xp, name)(self.local, axis=0) + self.row_offset
        best = self.comm.extreme(vals, op)
        hit = vals == best
        if np.dtype(self.dtype).kind == "f":
            hit = hit | (xp.isnan(vals) & xp.isnan(best))
        if self.local.shape[0] == 0:
            cand = rows
        else:
            cand = xp.where(hit, rows, xp.full(lane_shape, big, dtype="i8"))
        res = self.comm.extreme(cand, "min")
        if keepdims:
            res = res.reshape((1,) + tuple(lane_shape))
        return res

    # the public functions of the package call this when they are handed a sharded array
    def __dpnp_sharded__(self, func, *args, **kwargs):
        if func in ("sum", "max", "min"):
            return self._reduce(func, *args, **kwargs)
        if func == "mean":
            return self._mean(*args, **kwargs)
        if func in ("argmax", "argmin"):
            return self._arg("max" if func == "argmax" else "min", *args, **kwargs)
        raise NotImplementedError(f"{func} of a sharded array")

    def sum(self, axis=None, dtype=None, keepdims=False):
        return self._reduce("sum", axis, dtype, keepdims)

    def max(self, axis=None, keepdims=False):
        return self._reduce("max", axis, None, keepdims)

    def min(self, axis=None, keepdims=False):
        return self._reduce("min", axis, None, keepdims)

    def mean(self, axis=None, keepdims=False):
        return self._mean(axis, keepdims)

    def argmax(self, axis=None, keepdims=False):
        return self._arg("max", axis, keepdims)

    def argmin(self, axis=None, keepdims=False):
        return self._arg("min", axis, keepdims)


def elementwise(name, *operands, **kwargs):
    """`name` (a function of the package taking arrays) applied slab-wise to operands of which at
    least one is sharded; used by the ufunc objects."""
    lead = next(i for i, o in enumerate(operands) if isinstance(o, ShardedArray))
    first = operands[lead]
    xp = _xp(first.local)
    args = [first.local if i == lead else first._operand(o) for i, o in enumerate(operands)]
    out = kwargs.get("out")
    if out is not None:
        if not isinstance(out, ShardedArray):
            raise TypeError("out= of a sharded operation must be a sharded array")
        kwargs["out"] = first._operand(out)
        getattr(xp, name)(*args, **kwargs)
        return out
    return first._new(getattr(xp, name)(*args, **kwargs))
