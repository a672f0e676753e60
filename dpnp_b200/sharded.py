"""Leading-axis sharding of arrays over the GPUs of one box, one process per GPU.

Elementwise work on identically sharded operands needs no communication.  A
reduction either keeps whole rows on one GPU (no exchange) or produces one
partial result per rank that is combined in a single step:

* sum over the sharded axis / over everything: all-gather of the partials and
  a local sum in rank order, so every rank gets bit-identical results that do
  not depend on the collective's internal ordering;
* max / min: all-reduce with MAX / MIN;
* argmax / argmin over everything: all-gather of (value, global flat index)
  pairs, then the first-occurrence rule (better value; ties -> smaller index).

The reference has no multi-device execution (arrays are tied to one queue,
dpnp/tensor/_compute_follows_data.pyx:67-160); this module is new functionality.
``torch.distributed`` provides the process group: NCCL over NVLink for device
arrays, gloo for host arrays (used by the CPU tests of this logic).
"""

from __future__ import annotations

import numpy as np


def shard_bounds(n: int, world_size: int, rank: int) -> tuple[int, int]:
    """Half-open range of leading-axis indices owned by `rank` (sizes differ by at most one)."""
    base, extra = divmod(int(n), int(world_size))
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def _dist():
    import torch.distributed as dist

    if not dist.is_initialized():
        raise RuntimeError("torch.distributed is not initialised")
    return dist


def _gather(x, group=None):
    """List of every rank's `x` as NumPy arrays (host input)."""
    import torch

    dist = _dist()
    t = torch.from_numpy(np.ascontiguousarray(x))
    t = t.reshape(-1) if t.dim() == 0 else t
    outs = [torch.empty_like(t) for _ in range(dist.get_world_size(group))]
    dist.all_gather(outs, t, group=group)
    return outs


def _on_queue_stream(arr):
    """Context in which torch enqueues on the array's own stream: the collective is then ordered
    with the library's kernels by the stream, and the host does not wait for either."""
    import torch

    q = arr.sycl_queue
    return torch.cuda.stream(torch.cuda.ExternalStream(q.stream, device=f"cuda:{q.device}"))


def _as_torch(arr):
    """torch tensor over the memory of a C-contiguous device array of the library."""
    import torch

    if not arr.flags.c_contiguous:
        raise ValueError("collectives need C-contiguous device arrays")
    dt = arr.dtype
    if dt.kind == "u" and dt.itemsize > 1:
        # torch has no wide unsigned collectives: move the bits as signed integers of the same size
        import dpnp_b200.tensor as dpt
        arr = dpt.usm_ndarray._view(arr.usm_data, arr._ptr, arr.shape, arr.strides, np.dtype(f"i{dt.itemsize}"),
                                    arr.sycl_queue)
    return torch.as_tensor(arr, device=f"cuda:{arr.sycl_queue.device}")


def allreduce_sum_ordered(partial, group=None):
    """Sum of the ranks' partials, computed on every rank from the same gathered rows in the
    same fixed order: all ranks get the same bits, whatever order the collective works in."""
    if isinstance(partial, np.ndarray) or np.isscalar(partial):
        outs = _gather(partial, group)
        acc = outs[0].numpy().copy()
        for o in outs[1:]:
            acc = acc + o.numpy()
        return acc.reshape(np.shape(partial))
    import dpnp_b200 as dp

    dist = _dist()
    world = dist.get_world_size(group)
    arr = partial.get_array() if hasattr(partial, "get_array") else partial
    gathered = dp.empty((world, max(arr.size, 1)), dtype=arr.dtype, sycl_queue=arr.sycl_queue)
    with _on_queue_stream(arr):
        dist.all_gather_into_tensor(_as_torch(gathered.get_array()).view(-1), _as_torch(arr).reshape(-1),
                                    group=group)
    return dp.sum(gathered, axis=0, dtype=arr.dtype).reshape(partial.shape)


def allreduce_extreme(partial, op="max", group=None):
    """Elementwise max/min of the ranks' partials (in place for device arrays)."""
    import torch

    dist = _dist()
    red = dist.ReduceOp.MAX if op == "max" else dist.ReduceOp.MIN
    if isinstance(partial, np.ndarray) or np.isscalar(partial):
        t = torch.from_numpy(np.ascontiguousarray(partial))
        dist.all_reduce(t, op=red, group=group)
        return t.numpy().reshape(np.shape(partial))
    arr = partial.get_array() if hasattr(partial, "get_array") else partial
    with _on_queue_stream(arr):
        dist.all_reduce(_as_torch(arr), op=red, group=group)
    return partial


def combine_arg_extreme(value, global_index, op="max", group=None):
    """Global argmax/argmin from each rank's (extreme value, global flat index of its first
    occurrence).  Inputs are host scalars/0-d arrays; returns (value, index) as NumPy scalars."""
    import torch

    dist = _dist()
    world = dist.get_world_size(group)
    v = np.asarray(value)
    pair = np.zeros(2, dtype=np.float64 if v.dtype.kind == "f" else np.int64)
    if v.dtype.kind == "f":
        # indices below 2^53 are exact in float64
        pair[0], pair[1] = float(v), float(int(global_index))
    else:
        pair[0], pair[1] = int(v), int(global_index)
    t = torch.from_numpy(pair)
    backend = dist.get_backend(group)
    if backend == "nccl":
        t = t.cuda()
    outs = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(outs, t, group=group)
    pairs = np.stack([o.cpu().numpy() for o in outs])
    best = 0
    for r in range(1, world):
        a, b = pairs[r], pairs[best]
        a_nan, b_nan = a[0] != a[0], b[0] != b[0]
        if a_nan or b_nan:
            better = a_nan and (not b_nan or a[1] < b[1])
        elif a[0] == b[0]:
            better = a[1] < b[1]
        else:
            better = a[0] > b[0] if op == "max" else a[0] < b[0]
        if better:
            best = r
    return v.dtype.type(pairs[best][0]), np.int64(pairs[best][1])


def arg_extreme_sharded(x, index_offset, op="max", group=None):
    """Global argmax/argmin of an array sharded along its leading axis: `x` is this rank's shard,
    `index_offset` the flat index of its first element in the whole array.  The local search, the
    read of the extreme value and both exchanges stay on the device and on the array's stream; the
    host reads the gathered (value, index) pairs once and applies the first-occurrence rule.
    Returns (value, index) as NumPy scalars."""
    import ctypes as C

    import dpnp_b200 as dp
    from dpnp_b200._lib import check, lib, typenum_of

    dist = _dist()
    world = dist.get_world_size(group)
    arr = x.get_array() if hasattr(x, "get_array") else x
    if not arr.flags.c_contiguous:
        raise ValueError("the shard must be C-contiguous")
    q = arr.sycl_queue
    idx = (dp.argmax if op == "max" else dp.argmin)(x)            # 0-d int64 on the device
    idx_arr = idx.get_array() if hasattr(idx, "get_array") else idx
    val = dp.empty((1,), dtype=arr.dtype, sycl_queue=q)
    check(lib.dpb_take_one(typenum_of(arr.dtype), C.c_void_p(arr._ptr), arr.size, C.c_void_p(idx_arr._ptr),
                           C.c_void_p(val.get_array()._ptr), C.c_void_p(q.stream)))
    gidx = dp.add(dp.reshape(idx, (1,)), int(index_offset))          # global flat index
    vals = dp.empty((world,), dtype=arr.dtype, sycl_queue=q)
    idxs = dp.empty((world,), dtype="i8", sycl_queue=q)
    with _on_queue_stream(arr):
        dist.all_gather_into_tensor(_as_torch(vals.get_array()), _as_torch(val.get_array()), group=group)
        dist.all_gather_into_tensor(_as_torch(idxs.get_array()), _as_torch(gidx.get_array()), group=group)
    v, i = vals.asnumpy(), idxs.asnumpy()                            # the one host read
    best = 0
    for r in range(1, world):
        a_nan, b_nan = v[r] != v[r], v[best] != v[best]
        if a_nan or b_nan:
            better = a_nan and (not b_nan or i[r] < i[best])
        elif v[r] == v[best]:
            better = i[r] < i[best]
        else:
            better = v[r] > v[best] if op == "max" else v[r] < v[best]
        if better:
            best = r
    return v[best], np.int64(i[best])
