"""Process groups for one box with several GPUs: one process per GPU.

Two layers, neither of which needs PyTorch:

* :class:`HostGroup` -- the ranks of a job talking over TCP on the loopback interface through
  rank 0.  It carries small host-side messages: the NCCL unique id at start-up, barriers, timing
  maxima, and the partial results of host arrays (NumPy) in the CPU tests of the sharding logic.
  The ranks find each other through the launcher's environment (``RANK``, ``WORLD_SIZE``,
  ``MASTER_ADDR``, ``MASTER_PORT`` as ``python -m torch.distributed.run`` and most launchers
  export them): rank 0 listens on a free port and publishes it in a file in the temporary
  directory named after the launcher process and ``MASTER_PORT``.
* :class:`Communicator` -- a host group plus, when a GPU is present, an NCCL communicator behind
  the C ABI (``dpb_comm_*``): ordered sums, NaN-propagating max/min and first-occurrence
  argmax/argmin of per-GPU partial results, enqueued on the library's stream.

The reference has no counterpart: its arrays live on one device
(dpnp/tensor/_compute_follows_data.pyx:67-160).
"""

from __future__ import annotations

import ctypes as C
import os
import pickle
import socket
import struct
import tempfile
import time

import numpy as np

from . import _lib
from ._lib import check, lib

__all__ = ["HostGroup", "Communicator", "find_nccl_library"]

_group_seq = [0]


def _parent_token() -> str:
    """Identifies the launcher: its pid and start time (same for every rank it started)."""
    ppid = os.getppid()
    start = ""
    try:
        with open(f"/proc/{ppid}/stat") as fh:
            start = fh.read().rsplit(")", 1)[1].split()[19]
    except (OSError, IndexError):
        pass
    return f"{ppid}_{start}"


def _recv_exact(sock, n):
    buf = bytearray()
    while len(buf) < n:
        chunk = sock.recv(n - len(buf))
        if not chunk:
            raise ConnectionError("a rank closed its connection")
        buf += chunk
    return bytes(buf)


def _send_msg(sock, payload: bytes):
    sock.sendall(struct.pack("<Q", len(payload)) + payload)


def _recv_msg(sock) -> bytes:
    (n,) = struct.unpack("<Q", _recv_exact(sock, 8))
    return _recv_exact(sock, n)


class HostGroup:
    """All-gather of byte strings among the ranks of one job (star through rank 0)."""

    def __init__(self, rank=None, world=None, addr=None, port=None, timeout=120.0):
        env = os.environ
        self.rank = int(env.get("RANK", "0")) if rank is None else int(rank)
        self.world = int(env.get("WORLD_SIZE", "1")) if world is None else int(world)
        if not 0 <= self.rank < self.world:
            raise ValueError(f"rank {self.rank} is not in a group of {self.world}")
        self._peers = []        # rank 0: sockets of ranks 1..world-1 (index rank-1)
        self._sock = None       # other ranks: socket to rank 0
        self.timeout = float(timeout)
        if self.world == 1:
            return
        addr = addr or env.get("MASTER_ADDR", "127.0.0.1")
        key = port if port is not None else env.get("MASTER_PORT", "0")
        seq = _group_seq[0]
        _group_seq[0] += 1
        path = os.path.join(tempfile.gettempdir(), f"dpnp_b200_rdzv_{_parent_token()}_{key}_{seq}")
        if self.rank == 0:
            srv = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
            srv.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
            srv.bind((addr, 0))
            srv.listen(self.world)
            srv.settimeout(self.timeout)
            tmp = f"{path}.{os.getpid()}"
            with open(tmp, "w") as fh:
                fh.write(str(srv.getsockname()[1]))
            os.replace(tmp, path)
            peers = {}
            try:
                while len(peers) < self.world - 1:
                    conn, _ = srv.accept()
                    conn.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
                    conn.settimeout(self.timeout)
                    (r, w) = struct.unpack("<ii", _recv_exact(conn, 8))
                    if w != self.world or not 0 < r < self.world or r in peers:
                        conn.close()
                        raise RuntimeError(f"rank {r} of a group of {w} tried to join a group of {self.world}")
                    peers[r] = conn
            except socket.timeout:
                raise RuntimeError(f"only {len(peers) + 1} of {self.world} ranks joined within {self.timeout:.0f} s") from None
            finally:
                srv.close()
                try:
                    os.unlink(path)
                except OSError:
                    pass
            self._peers = [peers[r] for r in range(1, self.world)]
        else:
            deadline = time.monotonic() + self.timeout
            port_no = None
            while port_no is None:
                try:
                    with open(path) as fh:
                        port_no = int(fh.read().strip())
                except (OSError, ValueError):
                    if time.monotonic() > deadline:
                        raise RuntimeError(f"rank 0 did not publish its address within {self.timeout:.0f} s") from None
                    time.sleep(0.01)
            s = socket.create_connection((addr, port_no), timeout=self.timeout)
            s.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
            s.settimeout(self.timeout)
            s.sendall(struct.pack("<ii", self.rank, self.world))
            self._sock = s

    def allgather(self, payload: bytes) -> list:
        """Every rank's `payload`, in rank order, on every rank."""
        if self.world == 1:
            return [payload]
        if self.rank == 0:
            parts = [payload] + [_recv_msg(p) for p in self._peers]
            blob = pickle.dumps(parts, protocol=pickle.HIGHEST_PROTOCOL)
            for p in self._peers:
                _send_msg(p, blob)
            return parts
        _send_msg(self._sock, payload)
        return pickle.loads(_recv_msg(self._sock))

    def allgather_object(self, obj) -> list:
        return [pickle.loads(b) for b in self.allgather(pickle.dumps(obj, protocol=pickle.HIGHEST_PROTOCOL))]

    def barrier(self) -> None:
        self.allgather(b"")

    def max_float(self, value: float) -> float:
        return max(struct.unpack("<d", b)[0] for b in self.allgather(struct.pack("<d", float(value))))

    def close(self) -> None:
        for s in self._peers + ([self._sock] if self._sock else []):
            try:
                s.close()
            except OSError:
                pass
        self._peers, self._sock = [], None


def find_nccl_library():
    """Path of libnccl.so.2: ``DPNP_B200_NCCL_LIB``, else the ``nvidia.nccl`` wheel if one is
    installed (found without importing anything), else None (the dynamic loader's default)."""
    p = os.environ.get("DPNP_B200_NCCL_LIB")
    if p:
        return p
    import importlib.util

    try:
        spec = importlib.util.find_spec("nvidia.nccl")
    except (ImportError, ValueError):
        spec = None
    if spec is not None and spec.submodule_search_locations:
        for d in spec.submodule_search_locations:
            cand = os.path.join(d, "lib", "libnccl.so.2")
            if os.path.exists(cand):
                return cand
    return None


def _combine_host(parts, op):
    """Fold NumPy partials in rank order (host arrays: the CPU tests of the sharding logic)."""
    acc = parts[0].copy()
    for p in parts[1:]:
        if op == "sum":
            acc = acc + p
        elif op == "max":
            acc = np.where((acc != acc) | (acc >= p), acc, p) if acc.dtype.kind == "f" else np.maximum(acc, p)
        else:
            acc = np.where((acc != acc) | (acc <= p), acc, p) if acc.dtype.kind == "f" else np.minimum(acc, p)
    return acc


class Communicator:
    """The ranks of one job: host messages always, NCCL combines when arrays live on a GPU."""

    def __init__(self, host: HostGroup | None = None, queue=None, device=None, device_side=True):
        """`host`: the host group (default: made from the launcher's environment).  `queue` /
        `device`: where this rank's arrays live (default: the GPU numbered ``LOCAL_RANK``).
        ``device_side=False`` makes a host-only communicator (NumPy partials)."""
        self.host = host if host is not None else HostGroup()
        self.rank, self.world = self.host.rank, self.host.world
        self._handle = None
        self.queue = queue
        if not device_side:
            return
        if queue is None and _lib.device_count() > 0:
            from .memory import get_default_queue, select_default_device

            if device is None:
                device = int(os.environ.get("LOCAL_RANK", str(self.rank))) % _lib.device_count()
            select_default_device(device)
            self.queue = get_default_queue(device)
        if self.queue is not None:
            self._init_device()

    # ------------------------------------------------------------------ set-up
    def _init_device(self):
        q = self.queue
        q.activate()
        ident = (C.c_char * 128)()
        if self.world > 1:
            path = find_nccl_library()
            check(lib.dpb_comm_load(path.encode() if path else None))
            if self.rank == 0:
                check(lib.dpb_comm_unique_id(ident))
            ids = self.host.allgather(bytes(ident.raw) if self.rank == 0 else b"")
            ident = (C.c_char * 128).from_buffer_copy(ids[0])
        h = C.c_void_p()
        check(lib.dpb_comm_init(self.rank, self.world, ident, C.byref(h)))
        self._handle = h
        self.peer_exchange = False
        if self.world > 1 and os.environ.get("DPNP_B200_PEER", "1") != "0":
            self._init_peer_mailboxes()

    def _init_peer_mailboxes(self):
        """One-kernel combines over peer memory where every GPU of the group can map the others'
        (same box, NVLink); otherwise the group keeps NCCL.  Every rank takes part in both host
        exchanges whatever happens locally, and the switch is thrown only if all ranks succeeded."""
        handle, where, ok = (C.c_char * 64)(), C.create_string_buffer(32), True
        try:
            check(lib.dpb_device_pci_bus_id(self.queue.device, where, 32))
            check(lib.dpb_comm_peer_export(self._handle, handle, 64, None))
        except (RuntimeError, ValueError, MemoryError):
            ok = False
        # one GPU per rank: kernels that wait for each other must never share a GPU
        places = self.host.allgather_object((socket.gethostname(), where.value))
        if len(set(places)) != self.world or len({h for h, _ in places}) != 1:
            ok = False
        handles = self.host.allgather(bytes(handle.raw) if ok else b"")
        if ok and all(len(x) == 64 for x in handles):
            try:
                check(lib.dpb_comm_peer_attach(self._handle, b"".join(handles), self.world))
            except (RuntimeError, ValueError):
                ok = False
        else:
            ok = False
        if all(self.host.allgather_object(ok)):
            check(lib.dpb_comm_peer_enable(self._handle, 1))
            self.peer_exchange = True

    def close(self):
        h, self._handle = self._handle, None
        if h is not None:
            try:
                lib.dpb_comm_destroy(h)
            except Exception:
                pass
        self.host.close()

    # ------------------------------------------------------------------ helpers
    @staticmethod
    def _usm(x):
        return x.get_array() if hasattr(x, "get_array") else x

    def _need_device(self):
        if self._handle is None:
            raise RuntimeError("this communicator has no GPU side (no CUDA device was visible when it was made)")

    def _like(self, arr):
        from .tensor._usmarray import usm_ndarray

        return usm_ndarray._new_dense(arr.shape, arr.dtype, arr.sycl_queue)

    def _wrap(self, like, res):
        from .dpnp_array import dpnp_array

        return dpnp_array._create_from_usm_ndarray(res) if isinstance(like, dpnp_array) else res

    # ------------------------------------------------------------------ combines
    def sum_ordered(self, partial):
        """Sum of the ranks' partials, added in rank order on every rank (same bits everywhere)."""
        if isinstance(partial, np.ndarray) or np.isscalar(partial):
            p = np.ascontiguousarray(partial)
            return _combine_host(self.host.allgather_object(p), "sum").reshape(np.shape(partial))
        self._need_device()
        arr = self._usm(partial)
        if not arr.flags.c_contiguous:
            raise ValueError("partials must be C-contiguous")
        out = self._like(arr)
        q = arr.sycl_queue
        q.activate()
        check(lib.dpb_comm_sum_ordered(self._handle, _lib.typenum_of(arr.dtype), C.c_void_p(arr._ptr),
                                       C.c_void_p(out._ptr), arr.size, C.c_void_p(q.stream)))
        return self._wrap(partial, out)

    def extreme(self, partial, op="max"):
        """Elementwise max / min over the ranks' partials, NaN propagating."""
        if isinstance(partial, np.ndarray) or np.isscalar(partial):
            p = np.ascontiguousarray(partial)
            return _combine_host(self.host.allgather_object(p), op).reshape(np.shape(partial))
        self._need_device()
        arr = self._usm(partial)
        if not arr.flags.c_contiguous:
            raise ValueError("partials must be C-contiguous")
        out = self._like(arr)
        q = arr.sycl_queue
        q.activate()
        check(lib.dpb_comm_extreme(self._handle, _lib.typenum_of(arr.dtype), 1 if op == "max" else 0,
                                   C.c_void_p(arr._ptr), C.c_void_p(out._ptr), arr.size, C.c_void_p(q.stream)))
        return self._wrap(partial, out)

    def arg_extreme(self, shard, local_index, index_offset, op="max"):
        """(value, global flat index) of the extreme of a flattened sharded array: `shard` is this
        rank's part, `local_index` the position of its own extreme (0-d int64 array; ignored for an
        empty shard), `index_offset` the flat index of the shard's first element.  First occurrence
        wins across shards; NaN is extreme.  Host arrays give NumPy scalars, device arrays give
        0-d device arrays (nothing is read back)."""
        if isinstance(shard, np.ndarray):
            flat = shard.reshape(-1)
            mine = None if flat.size == 0 else (flat[int(local_index)], int(local_index) + int(index_offset))
            best = None
            for cand in self.host.allgather_object(mine):
                if cand is None:
                    continue
                if best is None:
                    best = cand
                    continue
                (v, i), (bv, bi) = cand, best
                vn, bn = v != v, bv != bv
                if vn or bn:
                    wins = vn and (not bn or i < bi)
                elif v == bv:
                    wins = i < bi
                else:
                    wins = v > bv if op == "max" else v < bv
                if wins:
                    best = cand
            if best is None:
                raise ValueError("reduction cannot be performed over zero-size axes")
            return best[0], np.int64(best[1])
        self._need_device()
        from .tensor._usmarray import usm_ndarray

        arr = self._usm(shard)
        if arr.size and not arr.flags.c_contiguous:
            raise ValueError("the shard must be C-contiguous")
        q = arr.sycl_queue
        li = self._usm(local_index) if arr.size else None
        val = usm_ndarray._new_dense((), arr.dtype, q)
        idx = usm_ndarray._new_dense((), np.dtype("i8"), q)
        q.activate()
        check(lib.dpb_comm_arg_extreme(self._handle, _lib.typenum_of(arr.dtype), 1 if op == "max" else 0,
                                       C.c_void_p(arr._ptr if arr.size else 0), arr.size,
                                       C.c_void_p(li._ptr if li is not None else 0), int(index_offset),
                                       C.c_void_p(val._ptr), C.c_void_p(idx._ptr), C.c_void_p(q.stream)))
        return self._wrap(shard, val), self._wrap(shard, idx)

    def allgather(self, local, counts=None):
        """Concatenation along axis 0 of the ranks' C-contiguous arrays (leading extents may
        differ; `counts` = every rank's leading extent, gathered over the host group if absent)."""
        if isinstance(local, np.ndarray):
            return np.concatenate(self.host.allgather_object(np.ascontiguousarray(local)), axis=0)
        self._need_device()
        from .tensor._usmarray import usm_ndarray

        arr = self._usm(local)
        if not arr.flags.c_contiguous:
            raise ValueError("shards must be C-contiguous")
        if counts is None:
            counts = self.host.allgather_object(arr.shape[0])
        row = int(np.prod(arr.shape[1:], dtype=np.int64)) * arr.dtype.itemsize
        most = max(counts)
        q = arr.sycl_queue
        q.activate()
        send = arr
        if arr.shape[0] != most:          # pad the short shards so that every rank sends the same size
            send = usm_ndarray._new_dense((most,) + arr.shape[1:], arr.dtype, q)
            check(lib.dpb_memcpy(C.c_void_p(send._ptr), C.c_void_p(arr._ptr), arr.shape[0] * row, 2,
                                 C.c_void_p(q.stream)))
        recv = usm_ndarray._new_dense((self.world * most,) + arr.shape[1:], arr.dtype, q)
        check(lib.dpb_comm_allgather(self._handle, C.c_void_p(send._ptr), C.c_void_p(recv._ptr), most * row,
                                     C.c_void_p(q.stream)))
        if all(c == most for c in counts):
            return self._wrap(local, recv)
        out = usm_ndarray._new_dense((sum(counts),) + arr.shape[1:], arr.dtype, q)
        at = 0
        for r, c in enumerate(counts):
            if c:
                check(lib.dpb_memcpy(C.c_void_p(out._ptr + at * row), C.c_void_p(recv._ptr + r * most * row),
                                     c * row, 2, C.c_void_p(q.stream)))
            at += c
        return self._wrap(local, out)

    def barrier(self):
        """Every rank has finished the work queued on its stream."""
        if self.queue is not None:
            self.queue.wait()
        self.host.barrier()
