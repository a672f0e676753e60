"""The chain compiler of ``dpnp_b200.fuse`` on the CPU: traced programs are run by a NumPy
emulation of the device interpreter's instruction set and compared, bit for bit, with the
same chain evaluated op by op in NumPy using the same elementary functions.  This checks the
graph building, common-subexpression sharing, instruction order, accumulator forwarding and
register allocation; the device interpreter itself is checked by the GPU tests."""

import math

import numpy as np
import pytest

import dpnp_b200 as dp
from dpnp_b200 import _fusion as F


def _erf(v):
    return np.array([math.erf(t) for t in np.asarray(v, dtype="f8").ravel()]).reshape(np.shape(v)).astype(v.dtype)


UNARY = {"negative": np.negative, "abs": np.abs, "exp": np.exp, "log": np.log, "sqrt": np.sqrt,
         "square": np.square, "reciprocal": np.reciprocal, "sin": np.sin, "cos": np.cos, "tanh": np.tanh,
         "expm1": np.expm1, "log1p": np.log1p, "floor": np.floor, "ceil": np.ceil, "sign": np.sign,
         "erf": _erf, "move": lambda v: v, "positive": lambda v: v}
BINARY = {"add": np.add, "subtract": np.subtract, "multiply": np.multiply, "divide": np.divide,
          "maximum": np.maximum, "minimum": np.minimum, "pow": np.power, "less": np.less,
          "less_equal": np.less_equal, "greater": np.greater, "greater_equal": np.greater_equal,
          "equal": np.equal, "not_equal": np.not_equal,
          "logical_and": lambda p, q: (p != 0) & (q != 0), "logical_or": lambda p, q: (p != 0) | (q != 0)}


def emulate(prog, inputs, n):
    """Executes the instruction words exactly as the device interpreter defines them."""
    dt = prog.dtype
    imm = [dt.type(v) for v in prog.imm[:max(1, prog.n_imm)]]
    regs, acc, outs = {}, None, {}
    # stores into an argument change what later reads of that argument see, as on the device
    inputs = [np.array(a, dtype=dt, copy=True) for a in inputs]

    def get(x, first):
        if x == 255:
            assert not first
            return acc
        if x >= 128:                      # an argument, read where it is used
            r = np.array(inputs[x - 128], dtype=dt, copy=True)
            return np.full(n, r.reshape(-1)[0], dt) if r.size == 1 else r.reshape(-1)
        if x >= 64:
            return np.full(n, imm[x - 64], dt)
        return regs[x]

    with np.errstate(all="ignore"):
        for pc, (op, dst, a, b, c) in enumerate(prog.listing()):
            first = pc == 0
            if op == "load":
                r = np.array(inputs[a], dtype=dt, copy=True)
                if r.size == 1:
                    r = np.full(n, r.reshape(-1)[0], dt)
            elif op == "store":
                outs[b] = get(a, first).copy()
                bind = prog.out_bind[b]
                if bind[0] == "slot" and bind[1] in prog.in_slots:
                    inputs[prog.in_slots.index(bind[1])] = outs[b].reshape(inputs[prog.in_slots.index(bind[1])].shape)
                continue
            elif op == "select":
                r = np.where(get(a, first) != 0, get(b, first), get(c, first))
            elif F._OPS[op] < F._FIRST_BINARY:
                r = UNARY[op](get(a, first))
            else:
                r = BINARY[op](get(a, first), get(b, first)).astype(dt)
            acc = r
            if dst != 255:
                assert dst < prog.n_reg
                regs[dst] = r
    return outs


class NumpyNamespace:
    """The functions a chain uses, on NumPy arrays (the op-by-op evaluation)."""
    erf = staticmethod(_erf)

    def __getattr__(self, name):
        return getattr(np, name)


def black_scholes(xp, price, strike, t, call, put, rate, vol):
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


def run_both(chain, arrays, scalars=(), outputs=0, dtype="f8"):
    """chain(xp, *arrays, *scalars); the last `outputs` arrays are written in place."""
    n = max(a.size for a in arrays)
    specs = [F.ArraySpec(dtype, a.shape) for a in arrays]
    fused = dp.fuse(lambda *args: chain(dp, *args))
    prog = fused.program(*specs, *scalars)
    assert prog is not None, fused.last_reason
    outs = emulate(prog, [arrays[s] for s in prog.in_slots], n)
    ref_arrays = [a.copy() for a in arrays]
    with np.errstate(all="ignore"):
        ref = chain(NumpyNamespace(), *ref_arrays, *scalars)
    return prog, outs, ref, ref_arrays


def test_black_scholes_chain_program():
    rng = np.random.default_rng(5)
    n = 4096
    P, S, T = rng.uniform(10, 50, n), rng.uniform(10, 50, n), rng.uniform(1, 2, n)
    call, put = np.zeros(n), np.zeros(n)
    prog, outs, _, ref = run_both(black_scholes, [P, S, T, call, put], (0.1, 0.2))
    # a - b is shared, T * mr is shared, no intermediate is stored; the arguments are read
    # where they are used and take no register
    ops = [l[0] for l in prog.listing()]
    assert ops.count("load") == 0 and ops.count("store") == 2 and len(prog.in_slots) == 3
    assert ops.count("subtract") == 4 and ops.count("erf") == 2 and ops.count("exp") == 1
    assert prog.n_reg <= 5
    assert [b for b in prog.out_bind] == [("slot", 3), ("slot", 4)]
    np.testing.assert_array_equal(outs[0], ref[3])
    np.testing.assert_array_equal(outs[1], ref[4])


def test_results_where_and_scalars():
    def chain(xp, x, y, s):
        m = xp.where((x > 0.5) & ~(y < -0.25), x * s, y - 2)
        lo = xp.minimum(xp.maximum(m, -1.0), 1.0)
        return lo, xp.sqrt(xp.abs(m)) + lo, +x

    rng = np.random.default_rng(6)
    x, y = rng.normal(0, 1, 1000).astype("f4"), rng.normal(0, 1, 1000).astype("f4")
    prog, outs, ref, _ = run_both(chain, [x, y], (3,), dtype="f4")
    assert prog.dtype == np.dtype("f4") and len(prog.out_bind) == 3
    for i, r in enumerate(ref):
        np.testing.assert_array_equal(outs[i], r.astype("f4"))


def test_read_then_write_of_the_same_argument_and_inplace_operators():
    def chain(xp, x, y):
        t = x * 2.0
        x[:] = y + 1.0          # x is written ...
        y += t                  # ... y is written from the OLD x
        return x * y            # and both new values are read back

    rng = np.random.default_rng(7)
    x, y = rng.normal(0, 1, 300), rng.normal(0, 1, 300)
    prog, outs, ref, ref_arrays = run_both(chain, [x, y])
    binds = prog.out_bind
    np.testing.assert_array_equal(outs[binds.index(("slot", 0))], ref_arrays[0])
    np.testing.assert_array_equal(outs[binds.index(("slot", 1))], ref_arrays[1])
    np.testing.assert_array_equal(outs[binds.index(("new",))], ref)
    # a store into an argument comes after the last instruction that reads that argument
    lst = prog.listing()
    for i, (op, dst, a, b, c) in enumerate(lst):
        if op == "store" and prog.out_bind[b][0] == "slot":
            code = 128 + prog.in_slots.index(prog.out_bind[b][1]) if prog.out_bind[b][1] in prog.in_slots else None
            assert all(code not in l[2:] for l in lst[i + 1:] if l[0] != "store")


def test_stores_that_copy_an_argument_another_store_overwrites():
    """A store whose value is an argument reads it when the store runs; a store into that
    argument must not run first."""
    def copy_then_overwrite(xp, a, b, c):
        c[:] = a
        a[:] = b * 2.0

    def rotate(xp, a, b):
        t = a + 0.0
        a[:] = b
        b[:] = t

    def swap(xp, a, b):
        ta, tb = +a, +b
        a[:] = tb
        b[:] = ta

    def old_value_returned(xp, a, b):
        t = +a
        a[:] = b * 3.0
        return t

    rng = np.random.default_rng(8)
    for chain, k in ((copy_then_overwrite, 3), (rotate, 2), (swap, 2), (old_value_returned, 2)):
        arrays = [rng.normal(0, 1, 130) for _ in range(k)]
        prog, outs, ref, ref_arrays = run_both(chain, arrays)
        for i, bind in enumerate(prog.out_bind):
            if bind[0] == "slot":
                np.testing.assert_array_equal(outs[i], ref_arrays[bind[1]], err_msg=chain.__name__)
            else:
                np.testing.assert_array_equal(outs[i], ref, err_msg=chain.__name__)


def test_size_one_arrays_broadcast_and_out_keyword():
    def chain(xp, x, s, out):
        xp.multiply(x, s, out=out)
        return xp.add(out, 1.0)

    x, s = np.linspace(-3, 3, 77), np.array([0.5])
    prog, outs, ref, ref_arrays = run_both(chain, [x, s, np.zeros(77)])
    assert prog.scalar_slots == [False, True, False]
    np.testing.assert_array_equal(outs[prog.out_bind.index(("slot", 2))], ref_arrays[2])
    np.testing.assert_array_equal(outs[prog.out_bind.index(("new",))], ref)


@pytest.mark.parametrize("seed", range(12))
def test_random_expression_graphs(seed):
    """Random DAGs with shared subexpressions: register reuse and accumulator forwarding
    must never change a value."""
    rng = np.random.default_rng(100 + seed)
    n_in, n_ops = int(rng.integers(1, 5)), int(rng.integers(5, 60))
    un = ["negative", "abs", "square", "sin", "cos", "tanh", "floor", "ceil", "sign"]
    bi = ["add", "subtract", "multiply", "maximum", "minimum"]
    plan = []
    for k in range(n_ops):
        if rng.random() < 0.3:
            plan.append(("u", un[rng.integers(len(un))], int(rng.integers(0, n_in + k))))
        elif rng.random() < 0.25:
            plan.append(("s", bi[rng.integers(len(bi))], int(rng.integers(0, n_in + k)),
                         float(np.round(rng.normal(), 2)), bool(rng.integers(2))))
        else:
            plan.append(("b", bi[rng.integers(len(bi))], int(rng.integers(0, n_in + k)),
                         int(rng.integers(0, n_in + k))))
    n_res = int(rng.integers(1, 4))
    picks = [int(v) for v in rng.integers(n_in, n_in + n_ops, n_res)]

    def chain(xp, *arrays):
        vals = list(arrays)
        for p in plan:
            if p[0] == "u":
                vals.append(getattr(xp, p[1])(vals[p[2]]))
            elif p[0] == "s":
                f = getattr(xp, p[1])
                vals.append(f(p[3], vals[p[2]]) if p[4] else f(vals[p[2]], p[3]))
            else:
                vals.append(getattr(xp, p[1])(vals[p[2]], vals[p[3]]))
        return tuple(vals[i] for i in picks)

    arrays = [rng.normal(0, 2, 257) for _ in range(n_in)]
    prog, outs, ref, _ = run_both(chain, arrays)
    assert prog.n_reg <= F._MAX_REG
    for t, r in zip(prog.results_tree[1], ref):
        assert t[0] == "node"
        np.testing.assert_array_equal(outs[prog.result_out[t[1]]], r)


def test_what_is_not_fused():
    spec = F.ArraySpec("f8", (10,))

    def no(fn, *args):
        f = dp.fuse(fn)
        assert f.program(*args) is None

    no(lambda x: x.sum(), spec)                                   # a reduction
    no(lambda x: x[1:] + 1.0, spec)                               # a view
    no(lambda x: x + 1 if x > 0 else x, spec)                     # data-dependent control flow
    no(lambda x: x > 0, spec)                                     # boolean result
    no(lambda x: (x > 0) + 1.0, spec)                             # arithmetic on a comparison
    no(lambda x, y: x + y, spec, F.ArraySpec("f4", (10,)))        # mixed types
    no(lambda x, y: x + y, spec, F.ArraySpec("f8", (5, 2)))       # different shapes
    no(lambda x: x + 1, F.ArraySpec("i4", (10,)))                 # integers
    no(lambda x: x * (1 << 60), spec)                             # scalar not exactly representable
    no(lambda x: x * np.float32(2), spec)                         # NumPy scalar of another type
    f = dp.fuse(lambda x: x * 2.0)
    assert f.program(spec) is not None


def test_specialised_source_has_one_statement_per_instruction_and_compiles():
    """The program written out as CUDA C++ for the run-time compiler: every instruction is one call
    of the operator class the per-op kernels use, in program order; with NVRTC present the source
    compiles for sm_100a on a machine without a GPU."""
    import ctypes as C

    from dpnp_b200 import _lib

    fused = dp.fuse(lambda *a: black_scholes(dp, *a, 0.1, 0.2))
    specs = [F.ArraySpec("f8", (4096,)) for _ in range(5)]
    prog = fused.program(*specs)
    assert prog is not None, fused.last_reason
    src = prog.source()
    body = src[src.index("__device__ __forceinline__ void chain("):src.index('extern "C" __global__')]
    statements = [ln.strip() for ln in body.splitlines() if ln.strip().startswith(("acc =", "y"))]
    listing = prog.listing()
    assert len(statements) == len(listing)
    classes = {"divide": "TrueDivideOp", "log": "LogOp", "multiply": "MultiplyOp", "sqrt": "SqrtOp",
               "subtract": "SubtractOp", "add": "AddOp", "erf": "ErfOp", "exp": "ExpOp"}
    for stmt, (name, dst, a, b, c3) in zip(statements, listing):
        if name == "store":
            assert stmt.startswith(f"y{b} =")
        else:
            assert classes[name] + "<T" in stmt, (stmt, name)
    assert src.count("ErfOp<T>::apply") == 2 and "typedef double T;" in src
    assert "const T x2" in src and "T &y1" in src                     # 3 inputs, 2 outputs
    f4 = dp.fuse(lambda x, s: dp.where(x > s, x, 0.5) * s)
    p4 = f4.program(F.ArraySpec("f4", (100,)), F.ArraySpec("f4", (1,)))
    assert p4 is not None, f4.last_reason
    s4 = p4.source()
    assert "typedef float T;" in s4 and "const T s1 = a.in[1][0];" in s4 and "GreaterOp<T, T>" in s4
    # NVRTC present (it ships with the CUDA toolkit): the source compiles without a device
    try:
        C.CDLL("libnvrtc.so.12")
    except OSError:
        pytest.skip("NVRTC is not installed here")
    assert prog.compile() > 10000 and p4.compile() > 1000
    # headers that cannot be found: the compiler's message comes back
    _lib.check(_lib.lib.dpb_fused_set_include_path(b"/nonexistent"))
    try:
        other = dp.fuse(lambda x: dp.cos(x) - 3.0).program(F.ArraySpec("f8", (10,)))
        with pytest.raises(RuntimeError, match="ew_ops.cuh"):
            other.compile()
    finally:
        _lib.check(_lib.lib.dpb_fused_set_include_path(None))
    with pytest.raises(ValueError):
        dp.fuse(lambda x: x, mode="fast")
