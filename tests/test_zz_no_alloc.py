"""The allocation-free row reduction (dpb_reduce_axis1_contig_noalloc).

It serves callers that must not allocate while they run (code embedded in a
framework that owns the device's memory, fixed-budget services): the partial
results of split rows live in an array inside the library image instead of the
pool.  Here it is called through the C ABI twice in a row and compared with the
pooled entry point, which partitions the work identically: integer results
must be equal, floating sums must agree within the tolerance of the other sum
tests (1e-5 / 1e-12 of the sum of magnitudes).  This file sorts last so that a
run stopping at the first failure has already executed every other test.
"""

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _run(fn, op, tin, tout, rows, cols, src, dst_dtype, stream):
    import dpnp_b200 as dp
    from dpnp_b200 import _lib

    out = dp.get_usm_ndarray(dp.empty(rows, dtype=dst_dtype))
    st = fn(_lib.REDUCE_OPS[op], _lib.typenum_of(tin), _lib.typenum_of(tout), rows, cols, src._ptr, 0, out._ptr, 0,
            stream)
    return st, out


@pytest.mark.parametrize("op,tin,tout,rows,cols", [
    ("sum", "f4", "f4", 3, 1 << 20), ("sum", "f8", "f8", 2, 300001), ("sum", "i4", "i8", 5, 1 << 19),
    ("max", "i4", "i4", 1, 1 << 22), ("min", "f4", "f4", 4, 70001), ("sum", "i8", "i8", 1000, 513),
])
def test_matches_pooled_entry_point_on_two_calls_in_a_row(op, tin, tout, rows, cols):
    import dpnp_b200 as dp
    from dpnp_b200 import _lib

    lib = _lib.lib
    rng = np.random.default_rng(rows * 31 + cols)
    host = (rng.normal(0, 1, (rows, cols)) * 100).astype(tin)
    src = dp.get_usm_ndarray(dp.asarray(host))
    stream = src.sycl_queue.stream
    st, ref = _run(lib.dpb_reduce_axis1_contig, op, tin, tout, rows, cols, src, tout, stream)
    _lib.check(st)
    ref = dp.asnumpy(ref)
    for _ in range(2):                      # the second call reuses whatever the first left in the scratch
        st, got = _run(lib.dpb_reduce_axis1_contig_noalloc, op, tin, tout, rows, cols, src, tout, stream)
        _lib.check(st)
        got = dp.asnumpy(got)
        if np.dtype(tout).kind == "f" and op == "sum":
            tol = 1e-5 if tout == "f4" else 1e-12
            mag = np.abs(host.astype(np.longdouble)).sum(axis=1)
            assert np.all(np.abs(got.astype(np.longdouble) - ref.astype(np.longdouble)) <= tol * mag)
            exact = host.astype(np.longdouble).sum(axis=1)
            assert np.all(np.abs(got.astype(np.longdouble) - exact) <= tol * mag)
        else:
            np.testing.assert_array_equal(got, ref)
    # a different reduction in between must not disturb the next one
    other = dp.get_usm_ndarray(dp.asarray(np.arange(1 << 20, dtype="i4")))
    st, o = _run(lib.dpb_reduce_axis1_contig_noalloc, "max", "i4", "i4", 1, 1 << 20, other, "i4", stream)
    _lib.check(st)
    assert int(dp.asnumpy(o)[0]) == (1 << 20) - 1


def test_refuses_what_does_not_fit_and_what_it_does_not_cover():
    import dpnp_b200 as dp
    from dpnp_b200 import _lib

    import ctypes as C

    lib = _lib.lib
    # The first refusal below relies on every row being split in two, which the partition does
    # when 64 blocks per SM exceed the 5000 rows: true from 79 SMs up.  On a smaller device the
    # call would not be refused and must not be made with the stand-in input.
    sms = C.c_int()
    _lib.check(lib.dpb_device_info(0, C.byref(sms), None, None, None))
    if sms.value * 64 <= 5000:
        pytest.skip("the refusal case is sized for devices with at least 79 SMs")
    src = dp.get_usm_ndarray(dp.empty((8,), dtype="f8"))     # never read: the calls are refused before any launch
    out = dp.get_usm_ndarray(dp.empty(5000, dtype="f8"))
    f8 = _lib.typenum_of("f8")
    # 5000 rows of 2^21 float64: with 64 blocks per SM every row is split in two, and
    # 5000 * 2 partials * 8 bytes = 80000 bytes exceed the 65536-byte built-in buffer
    _lib.check(lib.dpb_set_tuning(b"ctas_per_sm", 64))
    try:
        st = lib.dpb_reduce_axis1_contig_noalloc(_lib.REDUCE_OPS["sum"], f8, f8, 5000, 1 << 21, src._ptr, 0,
                                                 out._ptr, 0, out.sycl_queue.stream)
        assert st == _lib.ERR_VALUE
        assert "80000 bytes of scratch" in _lib.last_error() and "holds 65536" in _lib.last_error()
    finally:
        _lib.check(lib.dpb_set_tuning(b"ctas_per_sm", 8))
    f2 = _lib.typenum_of("f2")
    st = lib.dpb_reduce_axis1_contig_noalloc(_lib.REDUCE_OPS["sum"], f2, f2, 4, 100, src._ptr, 0, out._ptr, 0,
                                             out.sycl_queue.stream)
    assert st == _lib.ERR_RUNTIME
