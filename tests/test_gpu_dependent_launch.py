"""The streaming kernels are launched with programmatic stream serialisation: a kernel may be set
up while the one before it in the stream drains, and waits for it before it reads.  Long chains in
which every launch consumes what the launch before produced -- within one kernel family and across
families (elementwise, reductions, row broadcasts, transposes), out of place and in place -- must
give the results of the same chains with the switch off, bit for bit, and NumPy's."""

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _chains(dp, x, y, m):
    dx, dy = dp.asarray(x), dp.asarray(y)
    for i in range(300):
        dx = dx * 1.0001 + dy
        if i % 50 == 49:
            dx = dx - dp.sum(dx) * 1e-9
    dz = dp.asarray(x)
    for _ in range(200):
        dp.add(dz, dy, out=dz)
        dp.multiply(dz, 0.999, out=dz)
    dacc = dp.asarray(m)
    for _ in range(60):
        dacc = dacc - dp.sum(dacc, axis=0) * 1e-3
        dacc = dp.copy((dacc.T - dp.max(dacc, axis=1)).T, order="C")
    return dx.asnumpy(), dz.asnumpy(), dacc.asnumpy()


@pytest.mark.parametrize("n", [1000, 4096, 100_000, 1 << 20])
def test_chains_of_dependent_launches(n):
    import dpnp_b200 as dp
    from dpnp_b200 import _lib

    rng = np.random.default_rng(n)
    x, y, m = rng.normal(0, 1, n), rng.normal(0, 1, n), rng.normal(0, 1, (257, 1027))
    try:
        _lib.check(_lib.lib.dpb_set_tuning(b"pdl", 1))
        on = _chains(dp, x, y, m)
        _lib.check(_lib.lib.dpb_set_tuning(b"pdl", 0))
        off = _chains(dp, x, y, m)
    finally:
        _lib.check(_lib.lib.dpb_set_tuning(b"pdl", 1))
    for a, b in zip(on, off):
        np.testing.assert_array_equal(a, b)
    z = x.copy()
    for _ in range(200):
        z += y
        z *= 0.999
    np.testing.assert_array_equal(on[1], z)
    ref = x.copy()
    for i in range(300):
        ref = ref * 1.0001 + y
        if i % 50 == 49:
            ref = ref - ref.sum() * 1e-9
    np.testing.assert_allclose(on[0], ref, rtol=1e-11, atol=1e-11)
