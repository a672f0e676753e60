"""The Python orchestration above the native calls, on the CPU: arrays are views over a stand-in
memory object, allocations come from a stand-in pool and every native call is replaced by a
recorder, so what is checked is what the host layer decides -- result type, shape, layout, which
operands reach the kernel with which strides.  The direct routes of the plain calls
(`f(x)`, `f(x, y)`, array with Python scalar) must decide exactly what the general route decides."""

import numpy as np
import pytest

import dpnp_b200 as dp
from dpnp_b200 import _lib, memory
from dpnp_b200.dpnp_array import dpnp_array
from dpnp_b200.tensor import _elementwise_funcs as ef
from dpnp_b200.tensor import _tensor_elementwise_impl as tei
from dpnp_b200.tensor import _tensor_impl as ti
from dpnp_b200.tensor import _tensor_reductions_impl as tri
from dpnp_b200.tensor._usmarray import _dense_strides, usm_ndarray


class _Mem:
    nbytes = 1 << 44
    ptr = _ptr = 4096


class _Block:
    at = [1 << 32]

    def __init__(self, nbytes, device, stream):
        _Block.at[0] += (int(nbytes) + 255) // 256 * 256 + 256
        self.ptr, self.nbytes = _Block.at[0], nbytes

    def release(self):
        pass


class _Sub(usm_ndarray):
    """Same array, another class: takes the general route of every function."""


@pytest.fixture
def recorder(monkeypatch):
    calls = []

    class Native:
        ArrayCore = staticmethod(lambda *a: tuple(a))       # the "core" is the argument tuple itself
        Block = _Block

        def __getattr__(self, name):
            return lambda *a: calls.append((name,) + a)

    nat = Native()
    queue = memory.StreamQueue(0, stream=7)
    _Mem.sycl_queue = queue
    monkeypatch.setattr(memory, "_native", nat)
    monkeypatch.setattr(_lib, "native", nat)
    import dpnp_b200.tensor._usmarray as um
    monkeypatch.setattr(um, "_native", nat)
    for mod in (tei, ti, tri):
        monkeypatch.setattr(mod, "_nat", nat)
    # the per-op functions captured the real module when they were made: rebuild them
    for name, op in _lib.BINARY_OPS.items():
        c, r, i = tei._make_binary(name, op)
        for obj in (getattr(ef, name, None), getattr(dp, {"pow": "power"}.get(name, name), None)):
            if obj is not None and hasattr(obj, "binary_fn_"):
                monkeypatch.setattr(obj, "binary_fn_", c)
                monkeypatch.setattr(obj, "binary_inplace_fn_", i)
    for name, op in _lib.UNARY_OPS.items():
        c, r = tei._make_unary(name, op)
        for obj in (getattr(ef, name, None), getattr(dp, name, None)):
            if obj is not None and hasattr(obj, "unary_fn_"):
                monkeypatch.setattr(obj, "unary_fn_", c)
    at = [1 << 20]

    def arr(shape, dt="f4", strides=None, cls=usm_ndarray):
        at[0] += 1 << 26
        return cls._view(_Mem, at[0], tuple(shape), tuple(strides or _dense_strides(tuple(shape))), np.dtype(dt), queue)

    return calls, arr


def _as_general(x):
    v = x._like(x._ptr, x._shape, x._strides)
    v.__class__ = _Sub
    return v


LAYOUTS = [((7, 5), None), ((7, 5), (1, 7)), ((1, 5), (100, 1)), ((7, 1, 5), None), ((6,), None), ((), None),
           ((0, 3), None), ((4, 6), (12, 2)), ((4, 6), (6, -1))]


@pytest.mark.parametrize("name", ["add", "multiply", "less", "divide", "maximum"])
def test_binary_direct_route_decides_what_the_general_route_decides(recorder, name):
    calls, arr = recorder
    fn = getattr(ef, name)
    checked = 0
    for dt in ("f4", "f8", "i4", "?", "c8", "u8"):
        for shape, strides in LAYOUTS:
            for shape2, strides2 in ((shape, strides), (shape, None)):
                a, b = arr(shape, dt, strides), arr(shape2, dt, strides2)
                try:
                    want = fn(_as_general(a), _as_general(b))
                except ValueError:
                    with pytest.raises(ValueError):
                        fn(a, b)
                    continue
                general_call = calls[-1]
                got = fn(a, b)
                assert (got.dtype, got.shape, got.strides, got._flags) == (want.dtype, want.shape, want.strides, want._flags), (dt, shape, strides, strides2)
                # the kernel got the same operands (op id, then the three views), up to the fresh result pointer
                assert calls[-1][0] == general_call[0] == "binary"
                assert calls[-1][1] == general_call[1]
                assert [c[1:] for c in calls[-1][2:4]] == [c[1:] for c in general_call[2:4]]
                assert calls[-1][4][1:] == general_call[4][1:]
                checked += 1
    assert checked >= 90


@pytest.mark.parametrize("name", ["exp", "negative", "abs", "isnan", "erf"])
def test_unary_direct_route(recorder, name):
    calls, arr = recorder
    fn = getattr(ef, name)
    for dt in ("f2", "f4", "f8", "i4", "c16", "?"):
        for shape, strides in LAYOUTS:
            a = arr(shape, dt, strides)
            try:
                want = fn(_as_general(a))
            except ValueError:
                with pytest.raises(ValueError):
                    fn(a)
                continue
            general_calls = len(calls)
            got = fn(a)
            assert (got.dtype, got.shape, got.strides, got._flags) == (want.dtype, want.shape, want.strides, want._flags), (name, dt, shape, strides)
            assert len(calls) - general_calls in (1, 2)        # a cast to a temporary first where promotion asks for it


def test_scalar_operands_take_the_array_type_and_a_stride_zero_view(recorder):
    calls, arr = recorder
    a = dpnp_array._create_from_usm_ndarray(arr((3, 4), "f4"))
    # the scalar arrays are made with a host-to-device copy on first use: stand in for that too
    import dpnp_b200.tensor._elementwise_common as ec

    made = []

    def fake_scalar(value, dtype, queue):
        v = arr((), dtype)
        made.append((value, np.dtype(dtype)))
        return v

    import pytest as _pytest
    mp = _pytest.MonkeyPatch()
    mp.setattr(ec, "_scalar_to_array", fake_scalar)
    ec._scalar_view_cache.clear()
    try:
        r = a * 2.0
        assert r.dtype == np.float32 and r.shape == (3, 4) and made == [(2.0, np.dtype("f4"))]
        name, op, x1, x2, out = calls[-1][:5]
        assert name == "binary" and x2[5] == (0, 0) and x2[4] == (3, 4)          # broadcast with stride 0
        r = 3 - a                                                                  # reflected: the scalar comes first
        assert calls[-1][2][5] == (0, 0) and calls[-1][3][5] == (4, 1)
        before = len(made)
        _ = a * 2.0                                                                # same value again: nothing new is made
        assert len(made) == before
        ai = dpnp_array._create_from_usm_ndarray(arr((5,), "i4"))
        r = ai * 2.5                                                               # general route: int array, float scalar
        assert r.dtype == np.float64
    finally:
        mp.undo()
        ec._scalar_view_cache.clear()


def test_reductions_allocate_and_permute_as_the_reference_does(recorder):
    calls, arr = recorder
    x = dpnp_array._create_from_usm_ndarray(arr((6, 7, 8), "f4"))
    r = dp.sum(x, axis=1)
    name, op, src, trailing, dst = calls[-1][:5]
    assert name == "reduce" and trailing == 1 and r.shape == (6, 8) and r.dtype == np.float32
    assert src[4] == (6, 8, 7) and src[5] == (56, 1, 8)             # reduced axis moved to the end, as a view
    r = dp.sum(x, axis=-1)
    assert calls[-1][2][4] == (6, 7, 8) and calls[-1][2][5] == (56, 8, 1)      # already last: the array itself
    r = dp.sum(x, axis=(0, 2), keepdims=True)
    assert r.shape == (1, 7, 1) and calls[-1][3] == 2
    xi = dpnp_array._create_from_usm_ndarray(arr((4, 9), "i4"))
    assert dp.sum(xi).dtype == np.int64 and dp.max(xi, axis=0).dtype == np.int32
    assert dp.argmax(xi, axis=-1).dtype == np.int64 and dp.argmax(xi).shape == ()
    with pytest.raises(TypeError):
        dp.argmax(xi, axis=(0, 1))
    with pytest.raises(ValueError, match="zero-size"):
        dp.max(dpnp_array._create_from_usm_ndarray(arr((0, 3), "f4")), axis=0)
