"""The device paths of dpnp_b200.sharded on one GPU: a one-rank NCCL group exercises the
collectives on the library's own stream, the ordered sum of gathered partials and the
device-side (value, index) exchange of the sharded argmax."""

import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def one_rank_group():
    import torch.distributed as dist

    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    dist.init_process_group("nccl", rank=0, world_size=1)
    yield dist
    dist.destroy_process_group()


def test_collectives_on_device_arrays(one_rank_group):
    import dpnp_b200 as dp
    from dpnp_b200 import sharded

    rng = np.random.default_rng(0)
    x = rng.normal(0, 1, (300, 257)).astype("f4")
    d = dp.asarray(x)
    part = dp.sum(d, axis=0)
    tot = sharded.allreduce_sum_ordered(part)
    np.testing.assert_array_equal(tot.asnumpy(), part.asnumpy())          # one rank: the partial itself
    assert tot.dtype == part.dtype and tot.shape == part.shape
    ip = dp.sum(dp.asarray(np.arange(12, dtype="i4").reshape(3, 4)), axis=0)
    np.testing.assert_array_equal(sharded.allreduce_sum_ordered(ip).asnumpy(), ip.asnumpy())
    m = dp.max(d, axis=0)
    assert sharded.allreduce_extreme(m, "max") is m
    np.testing.assert_array_equal(m.asnumpy(), x.max(axis=0))
    scalar = dp.sum(d)
    np.testing.assert_array_equal(sharded.allreduce_sum_ordered(scalar).asnumpy(), scalar.asnumpy())


@pytest.mark.parametrize("dt", ["i4", "f8", "u1"])
def test_sharded_arg_extreme_keeps_value_and_index_on_the_device(one_rank_group, dt):
    import dpnp_b200 as dp
    from dpnp_b200 import _lib, sharded

    rng = np.random.default_rng(1)
    x = rng.integers(0, 100, (7, 5000)).astype(dt)             # many ties: first occurrence wins
    d = dp.asarray(x)
    v, i = sharded.arg_extreme_sharded(d, 1000, "max")
    assert v == x.max() and i == 1000 + int(x.argmax())
    v, i = sharded.arg_extreme_sharded(d, 0, "min")
    assert v == x.min() and i == int(x.argmin())
    if dt == "f8":
        x[3, 17] = np.nan                                      # NaN is the extreme
        v, i = sharded.arg_extreme_sharded(dp.asarray(x), 5, "max")
        assert np.isnan(v) and i == 5 + 3 * 5000 + 17
    # the element read used by it
    out = dp.empty((1,), dtype=dt)
    idx = dp.asarray(np.array([12345], dtype="i8"))
    import ctypes as C
    _lib.check(_lib.lib.dpb_take_one(_lib.typenum_of(np.dtype(dt)), C.c_void_p(d.get_array()._ptr), d.size,
                                     C.c_void_p(idx.get_array()._ptr), C.c_void_p(out.get_array()._ptr),
                                     C.c_void_p(d.sycl_queue.stream)))
    assert out.asnumpy()[0] == x.reshape(-1)[12345] or (dt == "f8" and np.isnan(out.asnumpy()[0]))
