"""``dpnp_b200.fuse`` on the device: a fused chain must give the bits of the same chain run
op by op (which the other GPU tests pin against the CPU oracle), in one launch.  Every test runs
with both executors of a fused program: the kernel compiled for the chain at run time and the
interpreter."""

import ctypes as C

import numpy as np
import pytest

from oracle import dpnp_oracle as orc

pytestmark = pytest.mark.gpu

KERNEL = {"compile": "ew_fused_specialized", "interpret": "ew_fused"}


@pytest.fixture(autouse=True, params=["compile", "interpret"])
def fuse_mode(request, monkeypatch):
    monkeypatch.setenv("DPNP_B200_FUSE", request.param)
    return request.param


def black_scholes(xp, price, strike, t, rate, vol, call, put):
    mr = -rate
    sig_sig_two = vol * vol * 2
    P, S, T = price, strike, t
    a = xp.log(P / S)
    b = T * mr
    z = T * sig_sig_two
    c = 0.25 * z
    y = 1.0 / xp.sqrt(z)
    w1 = (a - b + c) * y
    w2 = (a - b - c) * y
    d1 = 0.5 + 0.5 * xp.erf(w1)
    d2 = 0.5 + 0.5 * xp.erf(w2)
    Se = xp.exp(b) * S
    r = P * d1 - Se * d2
    call[:] = r
    put[:] = r - P + Se


@pytest.mark.parametrize("n", [1, 5, 1023, 1024, 1025, 4099, 1 << 20])
def test_black_scholes_fused_equals_op_by_op(n, fuse_mode):
    import dpnp_b200 as dp
    from dpnp_b200 import _lib

    rng = np.random.default_rng(n)
    P, S, T = rng.uniform(10, 50, n), rng.uniform(10, 50, n), rng.uniform(1, 2, n)
    dP, dS, dT = dp.asarray(P), dp.asarray(S), dp.asarray(T)
    call0, put0 = dp.empty(n), dp.empty(n)
    black_scholes(dp, dP, dS, dT, 0.1, 0.2, call0, put0)
    fused = dp.fuse(lambda *a: black_scholes(dp, *a))
    call1, put1 = dp.zeros(n), dp.zeros(n)
    _lib.reset_launch_count()
    fused(dP, dS, dT, 0.1, 0.2, call1, put1)
    assert fused.fused_calls == 1, fused.last_reason
    assert _lib.launch_count() == 1 and _lib.last_kernel() == KERNEL[fuse_mode]
    assert fused.last_executor == {"compile": "specialized", "interpret": "interpreted"}[fuse_mode]
    np.testing.assert_array_equal(call1.asnumpy(), call0.asnumpy())
    np.testing.assert_array_equal(put1.asnumpy(), put0.asnumpy())
    # and the chain itself is within the oracle's tolerance of the exact values
    c, p = orc.black_scholes_chain(P, S, T, 0.1, 0.2)
    np.testing.assert_allclose(call1.asnumpy(), c, rtol=1e-12, atol=1e-12)
    np.testing.assert_allclose(put1.asnumpy(), p, rtol=1e-12, atol=1e-12)
    # other scalars: a new program, same function object
    fused(dP, dS, dT, 0.05, 0.3, call1, put1)
    black_scholes(dp, dP, dS, dT, 0.05, 0.3, call0, put0)
    np.testing.assert_array_equal(call1.asnumpy(), call0.asnumpy())
    assert fused.fused_calls == 2


def test_float32_chain_with_where_results_and_special_values():
    import dpnp_b200 as dp

    def chain(x, y, s):
        m = dp.where((x > 0.5) & ~(y < -0.25), x * s, y - 2)
        lo = dp.minimum(dp.maximum(m, -1.0), 1.0)
        return lo, dp.sqrt(dp.abs(m)) + lo, dp.log(x) / dp.tanh(y), +x

    rng = np.random.default_rng(11)
    n = 3001
    x, y = rng.normal(0, 1, n).astype("f4"), rng.normal(0, 1, n).astype("f4")
    x[:6] = [np.nan, np.inf, -np.inf, 0.0, -0.0, 1.0]
    y[:6] = [1.0, np.nan, 0.0, -0.0, np.inf, -np.inf]
    dx, dy = dp.asarray(x), dp.asarray(y)
    ref = chain(dx, dy, 3)
    fused = dp.fuse(chain)
    got = fused(dx, dy, 3)
    assert fused.fused_calls == 1, fused.last_reason
    assert isinstance(got, tuple) and len(got) == 4
    for g, r in zip(got, ref):
        assert g.dtype == np.dtype("f4") and g.shape == (n,)
        np.testing.assert_array_equal(g.asnumpy().view("u4"), r.asnumpy().view("u4"))
    assert got[3] is not dx          # +x is a copy, as it is op by op


def test_unaligned_starts_2d_shapes_scalar_arrays_and_aliases():
    import dpnp_b200 as dp

    @dp.fuse
    def f(x, y, s, out):
        t = x * 2.0
        x[:] = y + s
        y += t
        dp.multiply(x, y, out=out)
        return out

    def ref(x, y, s, out):
        t = x * 2.0
        x[:] = y + s
        y += t
        dp.multiply(x, y, out=out)
        return out

    rng = np.random.default_rng(12)
    base = [rng.normal(0, 1, 5000) for _ in range(3)]
    for lo, shape in ((1, (4999,)), (0, (50, 100)), (3, (13, 7, 11))):
        size = int(np.prod(shape))
        mk = lambda: [dp.asarray(b)[lo:lo + size].reshape(shape) for b in base]
        s = dp.asarray(np.array([0.75]))
        a0, a1 = mk(), mk()
        r1 = f(*a1[:2], s, a1[2])
        assert f.last_reason is None, f.last_reason
        r0 = ref(*a0[:2], s, a0[2])
        assert r1 is a1[2]
        for u, v in zip(a0, a1):
            np.testing.assert_array_equal(u.asnumpy(), v.asnumpy())
    # the same array passed twice is one input
    x = dp.asarray(base[0])
    g = dp.fuse(lambda a, b: a * b + a)
    np.testing.assert_array_equal(g(x, x).asnumpy(), (x * x + x).asnumpy())
    assert g.fused_calls == 1


def test_stores_that_copy_an_argument_another_store_overwrites():
    """`c[:] = a; a[:] = ...`, a rotation through a temporary, a swap and an old value handed
    back: the fused launch must leave what the op-by-op evaluation leaves."""
    import dpnp_b200 as dp

    def copy_then_overwrite(a, b, c):
        c[:] = a
        a[:] = b * 2.0

    def rotate(a, b):
        t = a + 0.0
        a[:] = b
        b[:] = t

    def swap(a, b):
        ta, tb = +a, +b
        a[:] = tb
        b[:] = ta

    def old_value_returned(a, b):
        t = +a
        a[:] = b * 3.0
        return t

    rng = np.random.default_rng(21)
    n = 5003
    for chain, k in ((copy_then_overwrite, 3), (rotate, 2), (swap, 2), (old_value_returned, 2)):
        host = [rng.normal(0, 1, n) for _ in range(k)]
        # op by op on host copies defines the answer (plain assignments and IEEE-exact products)
        want = [h.copy() for h in host]
        want_res = chain(*want)
        dev = [dp.asarray(h) for h in host]
        fused = dp.fuse(chain)
        got_res = fused(*dev)
        assert fused.fused_calls == 1, (chain.__name__, fused.last_reason)
        for d, w in zip(dev, want):
            np.testing.assert_array_equal(d.asnumpy(), w, err_msg=chain.__name__)
        if want_res is not None:
            np.testing.assert_array_equal(got_res.asnumpy(), want_res, err_msg=chain.__name__)


def test_calls_that_are_not_fused_run_op_by_op():
    import dpnp_b200 as dp
    from dpnp_b200 import _lib

    f = dp.fuse(lambda x, y: x * y + 1)
    xi = dp.asarray(np.arange(10, dtype="i4"))
    np.testing.assert_array_equal(f(xi, xi).asnumpy(), np.arange(10) ** 2 + 1)
    assert f.eager_calls == 1 and "dtype" in f.last_reason
    x = dp.asarray(np.arange(12.0).reshape(3, 4))
    np.testing.assert_array_equal(f(x.T, x.T).asnumpy(), (np.arange(12.0).reshape(3, 4).T ** 2 + 1))
    assert f.eager_calls == 2 and "contiguous" in f.last_reason
    np.testing.assert_array_equal(f(x, x[0]).asnumpy(), x.asnumpy() * x.asnumpy()[0] + 1)   # broadcasting
    assert f.eager_calls == 3
    g = dp.fuse(lambda x: x / dp.sum(x))
    np.testing.assert_allclose(g(x).asnumpy(), x.asnumpy() / 66.0, rtol=1e-15)
    assert g.eager_calls == 1 and g.fused_calls == 0
    h = dp.fuse(lambda x, o: dp.add(x[1:], 1.0, out=o[1:]))          # overlapping is fine op by op
    o = dp.zeros((3, 4))
    h(x, o)
    assert h.eager_calls == 1
    # overlapping distinct arguments are never fused
    k = dp.fuse(lambda a, b: a + b)
    flat = dp.asarray(np.arange(20.0))
    np.testing.assert_array_equal(k(flat[:10], flat[5:15]).asnumpy(), np.arange(10.0) + np.arange(5.0, 15.0))
    assert "overlapping" in k.last_reason
    assert _lib.last_kernel() not in KERNEL.values()


def test_c_abi_rejects_malformed_programs():
    from dpnp_b200 import _fusion as F, _lib
    import dpnp_b200 as dp

    x, o = dp.asarray(np.arange(8.0)), dp.zeros(8)
    S = C.c_void_p(x.get_array().sycl_queue.stream)

    def run(words, n_reg=1, n_imm=0, typenum=11, n_in=1, n_out=1):
        code = (C.c_uint64 * len(words))(*words)
        imm = (C.c_double * 1)(2.0)
        ins = (C.c_void_p * 1)(x.get_array()._ptr)
        outs = (C.c_void_p * 1)(o.get_array()._ptr)
        prog = F.dpb_fused_program(typenum, len(words), n_reg, n_imm, n_in, n_out, code, imm, ins, None, outs)
        return _lib.lib.dpb_fused_elementwise(C.byref(prog), 8, S)

    ops = F._OPS
    w = lambda op, dst=255, a=0, b=0, c=0: ops[op] | dst << 8 | a << 16 | b << 24 | c << 32
    good = [w("load", 0, 0), w("multiply", 255, 0, 64), w("store", 255, 255, 0)]
    assert run(good, n_imm=1) == _lib.OK
    np.testing.assert_array_equal(o.asnumpy(), np.arange(8.0) * 2)
    bad = [
        [w("multiply", 0, 255, 0)],                       # accumulator before any instruction
        [w("load", 0, 1)],                                # input index out of range
        [w("load", 3, 0)],                                # register out of range
        [w("load", 0, 0), w("add", 0, 0, 65)],            # immediate out of range
        [w("load", 0, 0), w("store", 255, 0, 1)],         # output index out of range
        [200],                                            # unknown opcode
    ]
    for words in bad:
        assert run(words, n_imm=1) == _lib.ERR_VALUE, words
        assert "malformed" in _lib.last_error()
    assert run(good, n_imm=1, typenum=5) == _lib.ERR_TYPE
    assert run(good, n_reg=25, n_imm=1) == _lib.ERR_VALUE


@pytest.mark.parametrize("seed", range(24))
def test_random_chains_fused_equal_op_by_op(seed):
    """Random expression graphs (shared subexpressions, scalars on either side, comparisons
    feeding where, stores into arguments): the interpreter must give the bits of the same
    graph evaluated one kernel per operation."""
    import dpnp_b200 as dp

    rng = np.random.default_rng(500 + seed)
    dt = "f8" if seed % 2 else "f4"
    n_in, n_ops = int(rng.integers(1, 5)), int(rng.integers(4, 70))
    un = ["negative", "abs", "square", "sin", "cos", "tanh", "floor", "ceil", "sign", "exp", "sqrt", "log1p", "erf"]
    bi = ["add", "subtract", "multiply", "divide", "maximum", "minimum"]
    plan = []
    for k in range(n_ops):
        r = rng.random()
        if r < 0.3:
            plan.append(("u", un[rng.integers(len(un))], int(rng.integers(0, n_in + k))))
        elif r < 0.5:
            plan.append(("s", bi[rng.integers(len(bi))], int(rng.integers(0, n_in + k)),
                         float(np.round(rng.normal(), 2)) or 0.5, bool(rng.integers(2))))
        elif r < 0.6:
            plan.append(("w", int(rng.integers(0, n_in + k)), int(rng.integers(0, n_in + k)),
                         int(rng.integers(0, n_in + k)), float(np.round(rng.normal(), 1))))
        else:
            plan.append(("b", bi[rng.integers(len(bi))], int(rng.integers(0, n_in + k)),
                         int(rng.integers(0, n_in + k))))
    picks = [int(v) for v in rng.integers(n_in, n_in + n_ops, int(rng.integers(1, 4)))]
    store_into = int(rng.integers(0, n_in)) if rng.random() < 0.5 else None

    def chain(*arrays):
        vals = list(arrays)
        for p in plan:
            if p[0] == "u":
                vals.append(getattr(dp, p[1])(vals[p[2]]))
            elif p[0] == "s":
                f = getattr(dp, p[1])
                vals.append(f(p[3], vals[p[2]]) if p[4] else f(vals[p[2]], p[3]))
            elif p[0] == "w":
                vals.append(dp.where(vals[p[1]] > p[4], vals[p[2]], vals[p[3]]))
            else:
                vals.append(getattr(dp, p[1])(vals[p[2]], vals[p[3]]))
        if store_into is not None:
            arrays[store_into][:] = vals[picks[0]]
        return tuple(vals[i] for i in picks)

    n = int(rng.choice([1000, 4099, 1 << 16]))
    host = [rng.normal(0, 2, n).astype(dt) for _ in range(n_in)]
    a0, a1 = [dp.asarray(h) for h in host], [dp.asarray(h) for h in host]
    with np.errstate(all="ignore"):
        ref = chain(*a0)
        fused = dp.fuse(chain)
        got = fused(*a1)
    if fused.fused_calls == 0:
        assert "limits" in fused.last_reason or "register" in fused.last_reason, fused.last_reason
        return
    ut = "u8" if dt == "f8" else "u4"
    for g, r in zip(got, ref):
        np.testing.assert_array_equal(g.asnumpy().view(ut), r.asnumpy().view(ut))
    for u, v in zip(a0, a1):
        np.testing.assert_array_equal(u.asnumpy().view(ut), v.asnumpy().view(ut))


def test_auto_mode_compiles_where_the_compiler_is_found_and_explicit_modes_are_checked(monkeypatch):
    import dpnp_b200 as dp
    from dpnp_b200 import _fusion, _lib

    monkeypatch.setenv("DPNP_B200_FUSE", "auto")
    x = dp.asarray(np.linspace(-2, 2, 1001))
    f = dp.fuse(lambda v: dp.exp(v) * 2.0 - v)
    want = (dp.exp(x) * 2.0 - x).asnumpy()
    np.testing.assert_array_equal(f(x).asnumpy(), want)
    assert f.last_executor == ("specialized" if _fusion.specialize_available() else "interpreted")
    # the decorator's own mode wins over the environment
    g = dp.fuse(lambda v: dp.exp(v) * 2.0 - v, mode="interpret")
    np.testing.assert_array_equal(g(x).asnumpy(), want)
    assert g.last_executor == "interpreted" and _lib.last_kernel() == "ew_fused"
    with pytest.raises(ValueError):
        dp.fuse(lambda v: v, mode="fast")
    # headers that cannot be found: "compile" reports the compiler's message, "auto" interprets
    _lib.check(_lib.lib.dpb_fused_set_include_path(b"/nonexistent"))
    try:
        h = dp.fuse(lambda v: dp.sin(v) + 1.0, mode="compile")
        with pytest.raises(RuntimeError, match="ew_ops.cuh"):
            h(x)
        k = dp.fuse(lambda v: dp.sin(v) + 1.0, mode="auto")
        np.testing.assert_array_equal(k(x).asnumpy(), (dp.sin(x) + 1.0).asnumpy())
        assert k.last_executor == "interpreted"
    finally:
        _lib.check(_lib.lib.dpb_fused_set_include_path(None))
