"""The sharding rules and the multi-rank combine logic on CPU: 2 and 3 ranks as child processes,
host (NumPy) shards, messages over the library's own TCP host group and over a gloo process
group of ``torch.distributed`` wrapped to the same interface."""

import os
import socket
import subprocess
import sys
import textwrap

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = textwrap.dedent("""
    import os, sys
    import numpy as np
    sys.path.insert(0, os.environ["REPO_ROOT"])
    import dpnp_b200 as dp
    from dpnp_b200 import sharded
    from dpnp_b200.memory import ExecutionPlacementError

    backend = os.environ["HOST_BACKEND"]
    if backend == "gloo":
        import torch.distributed as dist

        class GlooGroup:
            # a gloo process group behind the interface of dpnp_b200._comm.HostGroup
            def __init__(self):
                dist.init_process_group(backend="gloo")
                self.rank, self.world = dist.get_rank(), dist.get_world_size()
            def allgather(self, payload):
                outs = [None] * self.world
                dist.all_gather_object(outs, payload)
                return outs
            allgather_object = allgather
            def barrier(self):
                dist.barrier()
            def max_float(self, v):
                return max(self.allgather(float(v)))
            def close(self):
                dist.destroy_process_group()
        host = GlooGroup()
    else:
        host = sharded.HostGroup()
    comm = sharded.Communicator(host, device_side=False)
    rank, world = comm.rank, comm.world
    rng = np.random.default_rng(0)                    # every rank builds the same global arrays

    # ---- low-level combines
    x = rng.normal(0, 1, (10, 257)).astype("f4")
    lo, hi = sharded.shard_bounds(x.shape[0], world, rank)
    mine = x[lo:hi]
    parts = [x[slice(*sharded.shard_bounds(10, world, r))] for r in range(world)]
    tot = comm.sum_ordered(mine.sum(axis=0))
    expect = parts[0].sum(axis=0)
    for p in parts[1:]:
        expect = expect + p.sum(axis=0)               # rank order, float32 adds
    assert tot.dtype == np.float32 and np.array_equal(tot, expect), "ordered sum"
    m = comm.extreme(np.asarray(mine.max()), "max")
    assert m == x.max()
    assert np.array_equal(comm.extreme(mine.min(axis=0), "min"), x.min(axis=0))
    withnan = mine.max(axis=0).copy()
    if rank == world - 1:
        withnan[3] = np.nan
    got = comm.extreme(withnan, "max")
    assert np.isnan(got[3]) and np.array_equal(np.delete(got, 3), np.delete(x.max(axis=0), 3))

    # ---- the wrapper: the same calls a single-device program makes
    xs = sharded.scatter_rows(x, comm)
    assert xs.shape == x.shape and xs.local.shape == mine.shape and "ShardedArray" in repr(xs)
    assert np.array_equal(xs.asnumpy(), x)
    y = dp.exp(xs) * 2.0 + xs                         # slabs: no exchange, result stays sharded
    assert isinstance(y, sharded.ShardedArray) and np.array_equal(y.asnumpy(), np.exp(x) * np.float32(2.0) + x)
    r1 = dp.sum(xs, axis=1)                           # rows whole on one rank: still sharded
    assert isinstance(r1, sharded.ShardedArray) and r1.shape == (10,)
    assert np.array_equal(r1.asnumpy(), np.concatenate([p.sum(axis=1) for p in parts]))
    r0 = dp.sum(xs, axis=0)                           # combined: a plain array, same on all ranks
    assert isinstance(r0, np.ndarray) and np.array_equal(r0, expect)
    assert dp.sum(xs, axis=0, keepdims=True).shape == (1, 257)
    full = dp.sum(xs)
    e = parts[0].sum()
    for p in parts[1:]:
        e = e + p.sum()
    assert np.array_equal(full, e)
    mean = dp.mean(xs)
    assert abs(float(mean) - float(x.astype("f8").mean())) < 1e-5
    assert np.array_equal(dp.max(xs, axis=0), x.max(axis=0)) and dp.min(xs) == x.min()
    assert np.array_equal(dp.max(xs, axis=1).asnumpy(), x.max(axis=1))
    # matrix minus row vector: the plain operand is the same on every rank
    assert np.array_equal((xs - x[0]).asnumpy(), x - x[0])
    # differently sharded operands and plain arrays spanning the sharded axis are refused
    other = sharded.scatter_rows(rng.normal(0, 1, (11, 257)).astype("f4"), comm)
    for bad in (lambda: xs + other, lambda: dp.add(xs, x), lambda: dp.multiply(x, xs)):
        try:
            bad()
        except ExecutionPlacementError:
            pass
        else:
            raise AssertionError("placement error expected")

    # ---- argmax / argmin with ties: first occurrence across shards
    xi = rng.integers(0, 4, (10, 50)).astype("i4")
    si = sharded.scatter_rows(xi, comm)
    assert int(dp.argmax(si)) == int(xi.argmax()) and int(dp.argmin(si)) == int(xi.argmin())
    assert np.array_equal(dp.argmax(si, axis=0), xi.argmax(axis=0))
    assert np.array_equal(dp.argmin(si, axis=0), xi.argmin(axis=0))
    assert np.array_equal(dp.argmax(si, axis=1).asnumpy(), xi.argmax(axis=1))
    xf = rng.normal(0, 1, (10, 50))
    xf[7, 3] = np.nan                                 # NaN is the extreme value, the first NaN wins
    xf[9, 3] = np.nan
    sf = sharded.scatter_rows(xf, comm)
    assert int(dp.argmax(sf)) == int(np.argmax(xf)) and int(dp.argmin(sf)) == int(np.argmin(xf))
    assert np.array_equal(dp.argmax(sf, axis=0), np.argmax(xf, axis=0))
    assert np.isnan(dp.max(sf))

    # ---- fewer rows than ranks: a rank with an empty shard still takes part in every combine
    tiny = rng.integers(0, 3, (world - 1, 6)).astype("i4")
    st = sharded.scatter_rows(tiny, comm)
    assert st.local.shape[0] == (1 if rank < world - 1 else 0)
    assert int(dp.argmax(st)) == int(tiny.argmax()) and int(dp.max(st)) == int(tiny.max())
    assert np.array_equal(dp.sum(st, axis=0), tiny.sum(axis=0))
    assert np.array_equal(dp.argmin(st, axis=0), tiny.argmin(axis=0))
    assert np.array_equal(dp.min(st, axis=0), tiny.min(axis=0))
    empty = sharded.scatter_rows(np.zeros((0, 4), dtype="f4"), comm)
    assert np.array_equal(dp.sum(empty, axis=0), np.zeros(4, dtype="f4"))
    for bad in (lambda: dp.max(empty), lambda: dp.argmax(empty)):
        try:
            bad()
        except ValueError:
            pass
        else:
            raise AssertionError("zero-size reduction must be refused")

    # ---- from_local checks the split
    ok = sharded.from_local(mine, comm)
    assert ok.shape == x.shape
    try:
        sharded.from_local(x[: 3 if rank == 0 else 1], comm)
    except ValueError:
        pass
    else:
        if world > 1:
            raise AssertionError("uneven shards must be refused")
    comm.barrier()
    comm.close()
    print("rank", rank, "ok")
""")


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_shard_bounds_cover_the_axis():
    from dpnp_b200 import sharded

    for n in (0, 1, 7, 8, 16384, 1000003):
        for world in (1, 2, 3, 8):
            spans = [sharded.shard_bounds(n, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1


def _run_ranks(tmp_path, world, backend, extra_env=None, script=WORKER):
    path = tmp_path / "worker.py"
    path.write_text(script)
    port = _free_port()
    procs = []
    for rank in range(world):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank),
                   MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), REPO_ROOT=ROOT, HOST_BACKEND=backend)
        env.update(extra_env or {})
        procs.append(subprocess.Popen([sys.executable, str(path)], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=240)[0] for p in procs]
    return procs, outs


@pytest.mark.parametrize("world,backend", [(2, "gloo"), (2, "tcp"), (3, "tcp")])
def test_sharded_arrays_and_combines_on_host_ranks(tmp_path, world, backend):
    procs, outs = _run_ranks(tmp_path, world, backend)
    for rank, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, f"rank {rank} failed:\n{out}"
        assert f"rank {rank} ok" in out


FAILING = textwrap.dedent("""
    import os, sys
    sys.path.insert(0, os.environ["REPO_ROOT"])
    from dpnp_b200 import sharded
    mode, rank = os.environ["FAIL_MODE"], int(os.environ["RANK"])
    try:
        if mode == "never_joins":
            if rank == 1:
                sys.exit(0)                            # this rank goes away before the group forms
            sharded.HostGroup(timeout=2.0)
        elif mode == "world_mismatch":
            sharded.HostGroup(world=3 if rank == 1 else 2, rank=rank, timeout=2.0)
    except (RuntimeError, ConnectionError, OSError) as exc:
        print("refused:", type(exc).__name__, exc)
        sys.exit(7)
    print("joined")
""")


@pytest.mark.parametrize("mode", ["never_joins", "world_mismatch"])
def test_group_formation_failures_are_errors_not_hangs(tmp_path, mode):
    """A rank that never arrives, or one that believes in another group size: the others get an
    exception within the timeout (failure made on the host; no GPU involved)."""
    procs, outs = _run_ranks(tmp_path, 2, "tcp", {"FAIL_MODE": mode}, FAILING)
    assert procs[0].returncode == 7 and "refused" in outs[0], outs


PEER_SETUP = textwrap.dedent("""
    import ctypes as C, os, sys, types
    sys.path.insert(0, os.environ["REPO_ROOT"])
    from dpnp_b200 import _comm, sharded

    mode, rank = os.environ["PEER_CASE"], int(os.environ["RANK"])
    calls = []

    class FakeLib:
        # stands where the native calls stand: records what the set-up asks for, fails where told to
        def dpb_device_pci_bus_id(self, device, buf, n):
            same = mode == "shared_gpu"
            buf.value = b"0000:17:00.0" if same else ("0000:%02x:00.0" % (0x17 + rank)).encode()
            return 0
        def dpb_comm_peer_export(self, handle, buf, cap, size):
            calls.append("export")
            if mode == "export_fails" and rank == 1:
                return 2
            C.memmove(buf, bytes([rank + 1]) * 64, 64)
            return 0
        def dpb_comm_peer_attach(self, handle, blob, count):
            calls.append(("attach", count, bytes(blob)[:1], bytes(blob)[64:65]))
            return 2 if (mode == "attach_fails" and rank == 0) else 0
        def dpb_comm_peer_enable(self, handle, on):
            calls.append(("enable", on))
            return 0
        def dpb_last_error(self):
            return b"stand-in failure"

    _comm.lib = FakeLib()
    comm = _comm.Communicator(sharded.HostGroup(timeout=20.0), device_side=False)
    comm._handle, comm.queue = C.c_void_p(1), types.SimpleNamespace(device=rank)
    comm.peer_exchange = False
    comm._init_peer_mailboxes()
    expect = mode == "all_good"
    assert comm.peer_exchange == expect, (mode, rank, comm.peer_exchange, calls)
    assert (("enable", 1) in calls) == expect, calls
    if mode in ("all_good", "attach_fails"):
        att = [c for c in calls if c[0] == "attach"][0]
        assert att[1:] == (2, b"\\x01", b"\\x02"), att            # both handles, in rank order
    if mode == "shared_gpu":
        assert not any(c[0] == "attach" for c in calls if isinstance(c, tuple)), calls
    comm.host.barrier()
    print("rank", rank, "ok")
""")


@pytest.mark.parametrize("case", ["all_good", "export_fails", "attach_fails", "shared_gpu"])
def test_peer_mailboxes_are_switched_on_by_all_ranks_or_by_none(tmp_path, case):
    """The set-up of the one-kernel combines is a collective decision made on the host: every rank
    takes part in both exchanges whatever happened locally, the switch is thrown only if every rank
    exported and attached, and never for two ranks on one GPU (their kernels would wait for each
    other on the same device).  The native calls are recording stand-ins; no GPU is involved."""
    procs, outs = _run_ranks(tmp_path, 2, "tcp", {"PEER_CASE": case}, PEER_SETUP)
    for rank, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, f"rank {rank} failed:\n{out}"
        assert f"rank {rank} ok" in out
