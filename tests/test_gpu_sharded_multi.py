"""Sharded reductions over two GPUs with real exchanges -- through the peer mailboxes (one kernel per
rank and combine) and through NCCL: one child process per GPU, no PyTorch.  Skipped where the box
shows fewer than two devices."""

import os
import socket
import subprocess
import sys
import textwrap

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = textwrap.dedent("""
    import os, sys
    import numpy as np
    sys.path.insert(0, os.environ["REPO_ROOT"])
    import dpnp_b200 as dp
    from dpnp_b200 import sharded

    from dpnp_b200 import _lib
    comm = sharded.init()
    rank, world = comm.rank, comm.world
    want_peer = os.environ.get("DPNP_B200_PEER", "1") != "0"
    assert comm.peer_exchange == want_peer, (comm.peer_exchange, want_peer)
    rng = np.random.default_rng(0)                    # the same global arrays on every rank
    x = rng.normal(0, 1, (1001, 4099)).astype("f4")
    xs = sharded.scatter_rows(x, comm)
    assert isinstance(xs.local, dp.ndarray) and xs.local.sycl_queue.device == rank

    # sum over the sharded axis: |got - exact| <= 1e-5 * sum|x| per column, identical on all ranks
    got = dp.sum(xs, axis=0).asnumpy()
    exact = x.astype(np.longdouble).sum(axis=0)
    mag = np.abs(x).astype(np.longdouble).sum(axis=0)
    assert np.all(np.abs(got.astype(np.longdouble) - exact) <= 1e-5 * mag)
    assert _lib.last_kernel() == ("comm_peer_sum_ordered" if want_peer else "comm_sum_ordered"), _lib.last_kernel()
    every = comm.host.allgather_object(got.tobytes())
    assert all(b == every[0] for b in every), "ranks disagree on the ordered sum"
    # and it is the rank-ordered float32 sum of the ranks' own partials
    parts = comm.host.allgather_object(dp.sum(xs.local, axis=0).asnumpy())
    acc = parts[0].copy()
    for p in parts[1:]:
        acc = acc + p
    np.testing.assert_array_equal(got, acc)
    tot = float(dp.sum(xs).asnumpy())
    assert abs(tot - float(x.astype(np.longdouble).sum())) <= 1e-5 * float(np.abs(x).sum())
    assert abs(float(dp.mean(xs).asnumpy()) - float(x.astype("f8").mean())) <= 1e-5 * float(np.abs(x).mean())
    np.testing.assert_array_equal(dp.sum(xs, axis=1).asnumpy(), np.concatenate(
        comm.host.allgather_object(dp.sum(xs.local, axis=1).asnumpy())))
    np.testing.assert_array_equal(dp.max(xs, axis=0).asnumpy(), x.max(axis=0))
    np.testing.assert_array_equal(dp.min(xs).asnumpy(), x.min())
    np.testing.assert_array_equal((dp.exp(xs) * 2.0).asnumpy()[::97], (dp.exp(dp.asarray(x[::97])) * 2.0).asnumpy())

    # ties everywhere: the first occurrence across shards wins
    xi = rng.integers(0, 1000, (64, 1 << 16)).astype("i4")
    si = sharded.scatter_rows(xi, comm)
    assert int(dp.argmax(si).asnumpy()) == int(xi.argmax())
    assert int(dp.argmin(si).asnumpy()) == int(xi.argmin())
    np.testing.assert_array_equal(dp.argmax(si, axis=0).asnumpy(), xi.argmax(axis=0))
    np.testing.assert_array_equal(dp.argmax(si, axis=1).asnumpy(), xi.argmax(axis=1))
    # the maximum planted on the LAST rank only, then also on the first: the index must move
    planted = xi.copy()
    planted[-1, 77] = 5000
    assert int(dp.argmax(sharded.scatter_rows(planted, comm)).asnumpy()) == planted.argmax() == 63 * (1 << 16) + 77
    planted[0, 123] = 5000
    assert int(dp.argmax(sharded.scatter_rows(planted, comm)).asnumpy()) == 123
    xf = rng.normal(0, 1, (10, 50))
    xf[7, 3] = np.nan
    xf[9, 3] = np.nan
    sf = sharded.scatter_rows(xf, comm)
    assert int(dp.argmax(sf).asnumpy()) == int(np.argmax(xf)) and np.isnan(dp.max(sf).asnumpy())
    np.testing.assert_array_equal(dp.argmax(sf, axis=0).asnumpy(), np.argmax(xf, axis=0))

    # fewer rows than ranks: the rank with the empty shard still joins every exchange
    tiny = rng.integers(0, 3, (world - 1, 6)).astype("i4")
    st = sharded.scatter_rows(tiny, comm)
    assert int(dp.argmax(st).asnumpy()) == int(tiny.argmax()) and int(dp.max(st).asnumpy()) == int(tiny.max())
    np.testing.assert_array_equal(dp.sum(st, axis=0).asnumpy(), tiny.sum(axis=0))
    np.testing.assert_array_equal(dp.argmin(st, axis=0).asnumpy(), tiny.argmin(axis=0))
    np.testing.assert_array_equal(st.asnumpy(), tiny)
    np.testing.assert_array_equal(xs.asnumpy(), x)
    # a payload beyond a mailbox slot (256 KiB per rank) takes the NCCL route on either setting
    wide = rng.normal(0, 1, (4, 100_000))
    sw = sharded.scatter_rows(wide, comm)
    gw = dp.sum(sw, axis=0)
    assert _lib.last_kernel() == "comm_sum_ordered", _lib.last_kernel()
    pw = comm.host.allgather_object(dp.sum(sw.local, axis=0).asnumpy())
    np.testing.assert_array_equal(gw.asnumpy(), pw[0] + pw[1])
    # many combines back to back: the two slot sets alternate and no call overtakes another
    outs = [dp.sum(xs * float(k), axis=0) for k in range(1, 41)]
    for k in (1, 17, 40):
        mine = dp.sum(xs.local * float(k), axis=0).asnumpy()
        ordered = None
        for part in comm.host.allgather_object(mine):
            ordered = part if ordered is None else ordered + part
        np.testing.assert_array_equal(outs[k - 1].asnumpy(), ordered)
    comm.barrier()
    comm.close()
    print("rank", rank, "ok")
""")


@pytest.mark.parametrize("peer", ["1", "0"], ids=["peer_mailboxes", "nccl"])
def test_two_gpus(tmp_path, peer):
    from dpnp_b200 import _lib

    if _lib.device_count() < 2:
        pytest.skip("needs two GPUs")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    procs = []
    for rank in range(2):
        # NVLS off: a rank that dies must not leave its memory bound to an NVLink switch group
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE="2", LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), REPO_ROOT=ROOT, NCCL_NVLS_ENABLE="0", DPNP_B200_PEER=peer)
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=600)[0] for p in procs]
    for rank, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, f"rank {rank} failed:\n{out}"
        assert f"rank {rank} ok" in out
