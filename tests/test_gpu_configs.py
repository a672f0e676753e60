"""The five benchmark configurations: parity with the oracle at sizes the oracle finishes in
seconds, and size-independent properties at the full sizes."""

import numpy as np
import pytest

from oracle import dpnp_oracle as orc

pytestmark = pytest.mark.gpu


def dev(x):
    import dpnp_b200 as dp

    return dp.asarray(x)


def test_c1_add_f32_2p24_bit_exact():
    import dpnp_b200 as dp

    rng = np.random.default_rng(0)
    a = rng.uniform(-1, 1, 1 << 24).astype("f4")
    b = rng.uniform(-1, 1, 1 << 24).astype("f4")
    got = dp.add(dev(a), dev(b))
    assert got.dtype == np.float32 and got.flags.c_contiguous
    np.testing.assert_array_equal(got.asnumpy(), a + b)


def bs_chain_device(dp, price, strike, t, rate, vol):
    call = dp.zeros(price.shape, dtype=price.dtype)
    put = -dp.ones(price.shape, dtype=price.dtype)
    r, pt = orc.black_scholes_chain(price, strike, t, rate, vol, xp=dp, erf=dp.erf)
    call[:] = r
    put[:] = pt
    return call, put


def test_c2_black_scholes_chain_and_fused():
    import dpnp_b200 as dp
    from dpnp_b200 import _lib

    n = 1 << 20
    rng = np.random.default_rng(7777777)
    p, k, t = rng.uniform(10, 50, n), rng.uniform(10, 50, n), rng.uniform(1, 2, n)
    dpp, dk, dt_ = dev(p), dev(k), dev(t)
    _lib.reset_launch_count()
    call, put = bs_chain_device(dp, dpp, dk, dt_, 0.1, 0.2)
    # 26 ufunc kernels of the chain, a fill and a negation for `put = -ones`; the two copies are
    # library memcpys and are not counted
    assert _lib.launch_count() == 28
    fc, fp = dp.empty(n), dp.empty(n)
    q = fc.sycl_queue
    _lib.check(_lib.lib.dpb_black_scholes_f64(n, dpp.get_array()._ptr, dk.get_array()._ptr, dt_.get_array()._ptr,
                                              0.1, 0.2, fc.get_array()._ptr, fp.get_array()._ptr, q.stream))
    # the fused kernel rounds every intermediate where the chain does
    np.testing.assert_array_equal(fc.asnumpy(), call.asnumpy())
    np.testing.assert_array_equal(fp.asnumpy(), put.asnumpy())
    # against the host chain: +,-,*,/,sqrt exact, exp/log/erf within ulps -> a few 1e-15 relative on the
    # intermediates; call/put are differences of products, hence the absolute term
    ec, ep = orc.black_scholes_chain(p, k, t, 0.1, 0.2)
    np.testing.assert_allclose(fc.asnumpy(), ec, rtol=1e-13, atol=1e-12)
    np.testing.assert_allclose(fp.asnumpy(), ep, rtol=1e-13, atol=1e-12)
    cc, cp = orc.black_scholes_c(p, k, t, 0.1, 0.2)
    np.testing.assert_allclose(fc.asnumpy(), cc, rtol=1e-13, atol=1e-12)
    # put-call parity holds for the computed values: call - put = P - S*exp(-rT)
    lhs = fc.asnumpy() - fp.asnumpy()
    np.testing.assert_allclose(lhs, p - k * np.exp(-0.1 * t), rtol=1e-12, atol=1e-11)


def test_c2_full_size_sample_against_the_oracle_and_the_fused_kernel():
    """2^26 options: the chain through the API, the `fuse` front-end and the hand-fused kernel give
    the same bits everywhere, and a sample (every 4099th option plus the first and last 4096)
    agrees with the CPU oracle on the same inputs."""
    import dpnp_b200 as dp
    from dpnp_b200 import _lib

    n = 1 << 26
    dp.random.seed(7777777)
    dpp, dk, dt_ = dp.random.uniform(10.0, 50.0, n), dp.random.uniform(10.0, 50.0, n), dp.random.uniform(1.0, 2.0, n)
    call, put = bs_chain_device(dp, dpp, dk, dt_, 0.1, 0.2)
    fc, fp = dp.empty(n), dp.empty(n)
    q = fc.sycl_queue
    _lib.check(_lib.lib.dpb_black_scholes_f64(n, dpp.get_array()._ptr, dk.get_array()._ptr, dt_.get_array()._ptr,
                                              0.1, 0.2, fc.get_array()._ptr, fp.get_array()._ptr, q.stream))
    assert bool(dp.all(fc == call)) and bool(dp.all(fp == put))
    chain = dp.fuse(lambda a, b, c: orc.black_scholes_chain(a, b, c, 0.1, 0.2, xp=dp, erf=dp.erf))
    uc, up = chain(dpp, dk, dt_)
    assert chain.fused_calls == 1, chain.last_reason
    assert bool(dp.all(uc == call)) and bool(dp.all(up == put))
    idx = np.unique(np.concatenate([np.arange(0, n, 4099), np.arange(4096), np.arange(n - 4096, n)]))
    take = lambda a: np.concatenate([a[:4096].asnumpy(), a[::4099].asnumpy(), a[n - 4096:].asnumpy()])
    hp, hk, ht = take(dpp), take(dk), take(dt_)
    ec, ep = orc.black_scholes_chain(hp, hk, ht, 0.1, 0.2)
    np.testing.assert_allclose(take(call), ec, rtol=1e-13, atol=1e-12)
    np.testing.assert_allclose(take(put), ep, rtol=1e-13, atol=1e-12)
    cc, cp = orc.black_scholes_c(hp, hk, ht, 0.1, 0.2)
    np.testing.assert_allclose(take(fc), cc, rtol=1e-13, atol=1e-12)
    np.testing.assert_allclose(take(fp), cp, rtol=1e-13, atol=1e-12)
    assert idx.size > 20000


def test_c3_sums_small_and_full_size():
    import dpnp_b200 as dp

    rng = np.random.default_rng(0)
    x = rng.normal(0, 1, (512, 65536)).astype("f4")
    d = dev(x)
    for ax in (1, 0, None):
        got = dp.sum(d, axis=ax).asnumpy()
        exact, mag = orc.sum_exact(x, axis=ax)
        assert np.all(np.abs(got.astype(np.longdouble) - exact) <= 1e-5 * mag)
    m = dp.mean(d).asnumpy()
    assert abs(float(m) - float(orc.sum_exact(x)[0] / x.size)) <= 1e-5 * float(orc.sum_exact(x)[1] / x.size)
    del d
    # full size 16384 x 65536 (4 GiB): sum of row sums == sum of column sums == total, within the
    # tolerance scaled by the sum of magnitudes; and linearity sum(2x) == 2 sum(x) exactly
    big = dp.random.normal(0, 1, (16384, 65536), dtype="f4")
    s1 = dp.sum(big, axis=1)
    s0 = dp.sum(big, axis=0)
    assert s1.shape == (16384,) and s0.shape == (65536,)
    tot = float(dp.sum(big).asnumpy())
    # sum of magnitudes measured on the device (float64 accumulation), not estimated
    mag = float(dp.sum(dp.abs(big), dtype="f8").asnumpy())
    assert 0.79 * big.size < mag < 0.81 * big.size             # E|N(0,1)| = 0.798
    t1 = float(np.sum(s1.asnumpy().astype("f8")))
    t0 = float(np.sum(s0.asnumpy().astype("f8")))
    # each of the three is within 1e-5 * sum|x| of the exact sum, hence within 2e-5 of one another;
    # they are asked to agree within the single bound
    assert abs(t1 - t0) <= 1e-5 * mag and abs(t1 - tot) <= 1e-5 * mag and abs(t0 - tot) <= 1e-5 * mag
    # and against the float64 sum of the same data
    exact = float(dp.sum(big, dtype="f8").asnumpy())
    assert abs(tot - exact) <= 1e-5 * mag and abs(t1 - exact) <= 1e-5 * mag and abs(t0 - exact) <= 1e-5 * mag
    big2 = big[:2048]
    np.testing.assert_array_equal(dp.sum(big2 * 2.0, axis=1).asnumpy(), 2.0 * dp.sum(big2, axis=1).asnumpy())
    np.testing.assert_allclose(float(dp.mean(big).asnumpy()), tot / (16384 * 65536), rtol=1e-6, atol=1e-9)


def test_c4_transposed_broadcast_multiply():
    import dpnp_b200 as dp
    from dpnp_b200 import _lib

    rng = np.random.default_rng(0)
    a = rng.uniform(-2, 2, (128, 512, 64)).astype("f4")          # reduced (1024, 4096, 64)
    b = np.random.default_rng(1).uniform(-2, 2, (64, 1, 512)).astype("f4")
    got = dp.multiply(dev(a).transpose(2, 0, 1), dev(b))
    assert got.shape == (64, 128, 512) and got.flags.c_contiguous
    np.testing.assert_array_equal(got.asnumpy(), a.transpose(2, 0, 1) * b)
    # full size: every out[i, j, k] must equal a[j, k, i] * b[i, 0, k]; checked exactly on the device with
    # the contiguous path (a copy of the transposed operand) as the independent route
    A = dp.random.uniform(-2, 2, (1024, 4096, 64), dtype="f4")
    B = dp.random.uniform(-2, 2, (64, 1, 4096), dtype="f4")
    out = dp.multiply(A.transpose(2, 0, 1), B)
    assert _lib.last_kernel().startswith("ew_transpose")
    ref = dp.multiply(dp.copy(A.transpose(2, 0, 1), order="C"), B)
    assert bool(dp.all(out == ref))
    sl = out[5, 100:102, :].asnumpy()
    np.testing.assert_array_equal(sl, A[100:102, :, 5].asnumpy() * B[5, 0, :].asnumpy())


def test_c5_max_argmax_with_many_ties():
    import dpnp_b200 as dp

    rng = np.random.default_rng(0)
    x = rng.integers(0, 1000, (8, 1 << 22)).astype("i4")
    d = dev(x)
    np.testing.assert_array_equal(dp.max(d).asnumpy(), x.max())
    np.testing.assert_array_equal(dp.max(d, axis=-1).asnumpy(), x.max(axis=-1))
    np.testing.assert_array_equal(dp.argmax(d).asnumpy(), x.argmax())
    np.testing.assert_array_equal(dp.argmax(d, axis=-1).asnumpy(), x.argmax(axis=-1))
    del d
    # full size (8, 2^29): the argmax must point at a maximum, and nothing before it may equal it
    big = dp.random.randint(0, 1000, (8, 1 << 29), dtype="i4")
    mx = dp.max(big, axis=-1).asnumpy()
    am = dp.argmax(big, axis=-1).asnumpy()
    assert (mx == 999).all()                                   # 2^29 draws from 1000 values
    flat = int(dp.argmax(big).asnumpy())
    assert flat == int(am[0]) and int(dp.max(big).asnumpy()) == 999
    for r in range(8):
        i = int(am[r])
        assert int(big[r, i].asnumpy()) == 999
        if i > 0:
            assert int(dp.max(big[r, :i]).asnumpy()) < 999
