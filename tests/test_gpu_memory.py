"""Allocator, streams and host<->device transfers."""

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_pool_reuses_memory_and_counts_bytes():
    import dpnp_b200 as dp
    from dpnp_b200 import memory

    q = dp.get_default_queue()
    a = dp.empty(1 << 20, dtype="f4")
    before = memory.pool_stats()
    del a
    b = dp.empty(1 << 20, dtype="f4")
    after = memory.pool_stats()
    assert after["reserved"] <= before["reserved"]      # the freed block is reused, not re-reserved
    assert after["used"] >= b.nbytes
    q.wait()
    assert b.get_array().usm_data.ptr % 256 == 0


def test_pool_limit_reports_out_of_memory_from_the_host():
    import dpnp_b200 as dp
    from dpnp_b200 import memory

    memory.pool_set_limit(1 << 20)
    try:
        with pytest.raises(MemoryError, match="pool limit"):
            dp.empty(1 << 22, dtype="f8")
    finally:
        memory.pool_set_limit(0)
    assert dp.empty(1 << 22, dtype="f8").size == 1 << 22


def test_free_is_ordered_after_pending_work():
    import dpnp_b200 as dp

    x = dp.random.uniform(0, 1, 1 << 24, dtype="f4")
    acc = dp.zeros(1 << 24, dtype="f4")
    for _ in range(20):
        t = x * 2.0          # temporaries are released while their kernels may still be queued
        acc += t
        del t
    np.testing.assert_allclose(acc.asnumpy(), 40.0 * x.asnumpy(), rtol=1e-6)


def test_round_trip_all_dtypes_and_layouts():
    import dpnp_b200 as dp

    rng = np.random.default_rng(0)
    for dt in ("?", "i1", "u2", "i4", "u8", "f2", "f4", "f8", "c8", "c16"):
        x = (rng.uniform(0, 100, (13, 7, 5))).astype(dt)
        for arr in (x, np.asfortranarray(x), x[::2, :, ::-1], x.T):
            d = dp.asarray(arr)
            assert d.shape == arr.shape and d.dtype == arr.dtype
            np.testing.assert_array_equal(d.asnumpy(), arr)
            np.testing.assert_array_equal(d.T.asnumpy(), arr.T)
    assert dp.asarray(np.asfortranarray(np.ones((3, 4)))).flags.f_contiguous
    assert dp.asarray([1, 2, 3]).dtype == np.int64 and dp.asarray([1.0]).dtype == np.float64
    assert dp.asarray(x).strides == x.strides                # byte strides at the dpnp level
    assert dp.get_usm_ndarray(dp.asarray(x)).strides == tuple(s // x.itemsize for s in x.strides)


def test_views_share_memory():
    import dpnp_b200 as dp

    x = dp.asarray(np.arange(24.0).reshape(2, 3, 4))
    v = x.transpose(2, 0, 1)
    v[0] = -1.0
    assert (x.asnumpy()[:, :, 0] == -1).all()
    r = x.reshape(6, 4)
    r[:, 1] = 5.0
    assert (x.asnumpy()[:, :, 1] == 5).all()
    with pytest.raises(ValueError):
        x.T.reshape(24, copy=False)
    np.testing.assert_array_equal(x.T.reshape(24).asnumpy(), x.asnumpy().T.reshape(24))
    np.testing.assert_array_equal(dp.broadcast_to(dp.asarray(np.arange(3.0)), (2, 3)).asnumpy(), np.broadcast_to(np.arange(3.0), (2, 3)))
    iface = x.__cuda_array_interface__
    assert iface["shape"] == (2, 3, 4) and iface["typestr"] == "<f8" and iface["strides"] is None


def test_random_fills():
    import dpnp_b200 as dp

    dp.random.seed(1)
    u = dp.random.uniform(10, 50, 1 << 20).asnumpy()
    assert u.min() >= 10 and u.max() < 50 and abs(u.mean() - 30) < 0.1
    dp.random.seed(1)
    np.testing.assert_array_equal(dp.random.uniform(10, 50, 1 << 20).asnumpy(), u)
    n = dp.random.normal(0, 1, 1 << 20, dtype="f4").asnumpy()
    assert abs(n.mean()) < 0.01 and abs(n.std() - 1) < 0.01
    i = dp.random.randint(0, 1000, 1 << 20, dtype="i4").asnumpy()
    assert i.min() == 0 and i.max() == 999
