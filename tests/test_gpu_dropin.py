"""User code written against dpnp runs unchanged: `import dpnp as np`."""

import os
import runpy

import numpy
import pytest

pytestmark = pytest.mark.gpu

# a checkout of the reference: DPNP_REFERENCE_ROOT, else a directory named "reference" beside this repository
REFERENCE_ROOT = os.environ.get("DPNP_REFERENCE_ROOT") or os.path.join(
    os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference")


def test_the_reference_example_file_runs_as_it_is(capsys):
    """examples/example_bs.py of the reference, executed unmodified with `dpnp` resolving to this
    library (skipped where no checkout of the reference is present)."""
    path = os.path.join(REFERENCE_ROOT, "examples", "example_bs.py")
    if not os.path.exists(path):
        pytest.skip("no checkout of the reference on this machine")
    import dpnp_b200

    ns = runpy.run_path(path, run_name="__main__")
    assert ns["np"] is dpnp_b200
    call, put = ns["call"], ns["put"]
    from oracle import dpnp_oracle as orc

    ec, ep = orc.black_scholes_chain(ns["price"].asnumpy(), ns["strike"].asnumpy(), ns["t"].asnumpy(),
                                     ns["RISK_FREE"], ns["VOLATILITY"])
    numpy.testing.assert_allclose(call.asnumpy(), ec, rtol=1e-13, atol=1e-12)
    numpy.testing.assert_allclose(put.asnumpy(), ep, rtol=1e-13, atol=1e-12)
    assert capsys.readouterr().out.count("[") >= 2


def test_example_style_program_runs_under_the_dpnp_name():
    import dpnp as np            # resolves to this library
    import dpnp_b200

    assert np is dpnp_b200
    size = 2**12
    dtype = np.default_float_type()
    np.random.seed(7777777)
    price = np.random.uniform(10.0, 50.0, size)
    strike = np.random.uniform(10.0, 50.0, size)
    t = np.random.uniform(1.0, 2.0, size)
    call = np.zeros(size, dtype=dtype)
    put = -np.ones(size, dtype=dtype)

    def black_scholes(price, strike, t, rate, vol, call, put):
        mr = -rate
        sig_sig_two = vol * vol * 2
        a = np.log(price / strike)
        b = t * mr
        z = t * sig_sig_two
        c = 0.25 * z
        y = 1.0 / np.sqrt(z)
        w1 = (a - b + c) * y
        w2 = (a - b - c) * y
        d1 = 0.5 + 0.5 * np.erf(w1)
        d2 = 0.5 + 0.5 * np.erf(w2)
        se = np.exp(b) * strike
        r = price * d1 - se * d2
        call[:] = r
        put[:] = r - price + se

    black_scholes(price, strike, t, 0.1, 0.2, call, put)
    assert isinstance(call, np.ndarray) and call.dtype == numpy.float64
    print(call[:10])
    print(put[:10])
    from oracle import dpnp_oracle as orc

    ec, ep = orc.black_scholes_chain(price.asnumpy(), strike.asnumpy(), t.asnumpy(), 0.1, 0.2)
    numpy.testing.assert_allclose(call.asnumpy(), ec, rtol=1e-13, atol=1e-12)
    numpy.testing.assert_allclose(put.asnumpy(), ep, rtol=1e-13, atol=1e-12)


def test_numpy_style_snippets():
    import dpnp as np

    a = np.asarray(numpy.arange(12, dtype="f4").reshape(3, 4))
    b = np.ones((4,), dtype="f4")
    assert (a + b).shape == (3, 4) and (a.T * 2).shape == (4, 3)
    assert float(np.sum(a)) == 66.0 and float(a.mean()) == 5.5
    assert int(np.argmax(a)) == 11 and a.max(axis=0).asnumpy().tolist() == [8.0, 9.0, 10.0, 11.0]
    assert np.where(a > 5, a, 0.0).asnumpy().sum() == 51.0
    out = np.empty_like(a)
    np.multiply(a, a, out=out)
    assert float(out[2, 3]) == 121.0
    assert repr(np.asarray([1.0, 2.0])).startswith("array(")
    assert (a[1:, ::2].asnumpy() == numpy.arange(12, dtype="f4").reshape(3, 4)[1:, ::2]).all()
    assert a.strides == (16, 4) and a.T.strides == (4, 16)
