"""The device side of the sharded reductions on one GPU: a one-rank communicator runs the gather
buffer, the ordered-sum / extreme kernels and the packed (value, index) exchange of the sharded
argmax on the library's own stream (a group of one needs no NCCL call).  The same code with real
exchanges runs in tests/test_gpu_sharded_multi.py where the box has two GPUs."""

import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def comm():
    from dpnp_b200 import sharded

    c = sharded.Communicator(sharded.HostGroup(rank=0, world=1))
    yield c
    c.close()


def test_combines_on_device_arrays(comm):
    import dpnp_b200 as dp

    rng = np.random.default_rng(0)
    x = rng.normal(0, 1, (300, 257)).astype("f4")
    d = dp.asarray(x)
    part = dp.sum(d, axis=0)
    tot = comm.sum_ordered(part)
    np.testing.assert_array_equal(tot.asnumpy(), part.asnumpy())          # one rank: the partial itself
    assert tot.dtype == part.dtype and tot.shape == part.shape and tot is not part
    for dt in ("i4", "u8", "f2", "f8", "c8", "?"):
        p = dp.asarray((rng.normal(0, 3, 1000) > 0.5).astype(dt) if dt == "?" else rng.normal(0, 3, 1000).astype(dt))
        np.testing.assert_array_equal(comm.sum_ordered(p).asnumpy(), p.asnumpy())
    m = dp.max(d, axis=0)
    np.testing.assert_array_equal(comm.extreme(m, "max").asnumpy(), x.max(axis=0))
    np.testing.assert_array_equal(comm.extreme(dp.min(d), "min").asnumpy(), x.min())
    big = dp.asarray(rng.normal(0, 1, 1 << 19))                          # 4 MiB: the gather buffer grows
    np.testing.assert_array_equal(comm.sum_ordered(big).asnumpy(), big.asnumpy())
    np.testing.assert_array_equal(comm.sum_ordered(part).asnumpy(), part.asnumpy())


@pytest.mark.parametrize("dt", ["i4", "f8", "u1", "f2", "c16"])
def test_sharded_arg_extreme_keeps_value_and_index_on_the_device(comm, dt):
    import dpnp_b200 as dp

    rng = np.random.default_rng(1)
    x = rng.integers(0, 100, (7, 5000)).astype(dt)             # many ties: first occurrence wins
    d = dp.asarray(x)
    v, i = comm.arg_extreme(d, dp.argmax(d), 1000, "max")
    assert v.shape == () and i.shape == () and i.dtype == np.int64
    assert v.asnumpy() == x.max() and int(i.asnumpy()) == 1000 + int(x.argmax())
    v, i = comm.arg_extreme(d, dp.argmin(d), 0, "min")
    assert v.asnumpy() == x.min() and int(i.asnumpy()) == int(x.argmin())
    if dt == "f8":
        x[3, 17] = np.nan                                      # NaN is the extreme
        d = dp.asarray(x)
        v, i = comm.arg_extreme(d, dp.argmax(d), 5, "max")
        assert np.isnan(v.asnumpy()) and int(i.asnumpy()) == 5 + 3 * 5000 + 17


def test_sharded_array_through_the_public_functions(comm):
    """One rank holds everything: every function must give what the plain array gives."""
    import dpnp_b200 as dp
    from dpnp_b200 import sharded

    rng = np.random.default_rng(2)
    x = rng.normal(0, 1, (64, 300)).astype("f4")
    xs = sharded.scatter_rows(x, comm)
    d = dp.asarray(x)
    assert isinstance(xs.local, dp.ndarray)
    y = dp.exp(xs) * 2.0 + xs
    np.testing.assert_array_equal(y.asnumpy(), (dp.exp(d) * 2.0 + d).asnumpy())
    np.testing.assert_array_equal(dp.sum(xs, axis=0).asnumpy(), dp.sum(d, axis=0).asnumpy())
    np.testing.assert_array_equal(dp.sum(xs, axis=1).asnumpy(), dp.sum(d, axis=1).asnumpy())
    np.testing.assert_array_equal(dp.sum(xs).asnumpy(), dp.sum(d).asnumpy())
    np.testing.assert_array_equal(dp.mean(xs).asnumpy(), dp.mean(d).asnumpy())
    np.testing.assert_array_equal(dp.max(xs, axis=0).asnumpy(), x.max(axis=0))
    assert int(dp.argmax(xs).asnumpy()) == int(x.argmax())
    np.testing.assert_array_equal(dp.argmin(xs, axis=0).asnumpy(), x.argmin(axis=0))
    np.testing.assert_array_equal(dp.argmax(xs, axis=1).asnumpy(), x.argmax(axis=1))
    assert dp.sum(xs, axis=0, keepdims=True).shape == (1, 300)
    with pytest.raises(dp.ExecutionPlacementError):
        dp.add(xs, d)


def test_communicator_errors(comm):
    from dpnp_b200 import _lib

    h = C.c_void_p()
    assert _lib.lib.dpb_comm_init(2, 2, None, C.byref(h)) != 0 and "rank 2" in _lib.last_error()
    assert _lib.lib.dpb_comm_init(0, 2, None, C.byref(h)) != 0 and "unique id" in _lib.last_error()
    junk = (C.c_char * 64)()
    assert _lib.lib.dpb_comm_sum_ordered(junk, 10, None, None, 4, None) != 0
    assert "not a communicator" in _lib.last_error()


def test_the_bounded_wait_of_the_peer_exchange_gives_up_and_reports_it(comm):
    """The peer-mailbox exchange waits for the other ranks' flags with a bounded number of probes.
    Here the wait is run on a flag that nothing sets: it must come back, say that it gave up, and
    leave the device and the communicator usable."""
    import dpnp_b200 as dp
    from dpnp_b200 import _lib

    lib, check = _lib.lib, _lib.check
    handle, size = (C.c_char * 64)(), C.c_int64()
    check(lib.dpb_comm_peer_export(comm._handle, handle, 64, C.byref(size)))
    assert size.value == 64
    q = dp.get_default_queue()
    for polls in (0, 1000):
        gave_up = C.c_int(-1)
        check(lib.dpb_comm_peer_probe_wait(comm._handle, polls, C.byref(gave_up), C.c_void_p(q.stream)))
        assert gave_up.value == 1 and _lib.last_kernel() == "comm_peer_probe_wait"
    with pytest.raises(ValueError):
        check(lib.dpb_comm_peer_export(comm._handle, handle, 8, None))              # room for the handle
    with pytest.raises(ValueError):
        check(lib.dpb_comm_peer_attach(comm._handle, bytes(64), 3))                  # one handle per rank
    x = dp.asarray(np.arange(12.0))
    np.testing.assert_array_equal(comm.sum_ordered(x).asnumpy(), np.arange(12.0))    # still in working order
