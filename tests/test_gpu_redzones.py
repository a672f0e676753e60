"""Guarded pool blocks as a stand-in for a memory checker: with the "redzones" switch on, every
block carries patterned bytes in front and behind which are verified when the block is freed.
Small-shape sweeps over every kernel family must leave the guard bytes intact, through the usual
kernel choice and through the generic kernels; a deliberate overrun that stays inside the library's
own allocation (16 bytes into the trailing guard zone) must be reported."""

import ctypes as C
import gc

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _report(lib, check):
    blocks, nbytes = C.c_int64(), C.c_int64()
    first = (C.c_int64 * 3)()
    check(lib.dpb_debug_redzone_report(C.byref(blocks), C.byref(nbytes), first))
    return blocks.value, nbytes.value, list(first)


@pytest.fixture
def guarded():
    from dpnp_b200 import _lib

    lib, check = _lib.lib, _lib.check
    gc.collect()
    _report(lib, check)                                    # clear what earlier tests may have left
    check(lib.dpb_set_tuning(b"redzones", 1))
    yield lib, check
    check(lib.dpb_set_tuning(b"redzones", 0))
    check(lib.dpb_set_tuning(b"force_generic", 0))


def _sweep(dp):
    rng = np.random.default_rng(0)
    for n in (1, 2, 3, 7, 31, 32, 33, 255, 256, 257, 1023, 1025, 4099):
        for dt in ("f4", "f8", "i2", "c8", "?"):
            a = dp.asarray((rng.uniform(-3, 3, n) > 0).astype(dt) if dt == "?" else rng.uniform(-3, 3, n).astype(dt))
            b = dp.asarray((rng.uniform(-3, 3, n) > 0).astype(dt) if dt == "?" else rng.uniform(1, 3, n).astype(dt))
            dp.add(a, b); dp.multiply(a[::-1], b); dp.equal(a, b); dp.where(a != b, a, b)
            if dt in ("f4", "f8"):
                dp.exp(a); dp.erf(a[::2]); dp.sum(a); dp.max(a); dp.argmax(a); dp.cumsum(a); a * 2.0
                for mode in ("compile", "interpret"):           # both executors of a fused chain
                    f = dp.fuse(lambda x, y: dp.sqrt(dp.abs(x)) * y + 1.0, mode=mode)
                    f(a, b)
    for shape in ((3, 5), (17, 33), (64, 65), (5, 7, 9), (33, 1, 31), (2, 129, 3)):
        x = dp.asarray(rng.normal(0, 1, shape).astype("f4"))
        y = dp.asarray(rng.normal(0, 1, shape[-1]).astype("f4"))
        dp.subtract(x, y); dp.multiply(x.T, 2.0); dp.add(x.T, x.T); dp.copy(x.T, order="C")
        dp.multiply(x.transpose(*reversed(range(x.ndim))), 1.5)
        for ax in list(range(x.ndim)) + [None, tuple(range(x.ndim - 1))]:
            dp.sum(x, axis=ax); dp.max(x, axis=ax); dp.mean(x, axis=ax)
            if not isinstance(ax, tuple):
                dp.argmin(x, axis=ax)
                dp.cumsum(x, axis=ax if ax is not None else None)
        dp.astype(x, "f8"); dp.astype(x[:, ::2], "i4")
    # the single-pass scan of long rows (opt-in), ragged last tile, and its repair launches
    from dpnp_b200 import _lib
    for polls in (1 << 20, 0):
        _lib.check(_lib.lib.dpb_set_tuning(b"scan_lookback_polls", polls))
        try:
            for shape, dt in (((70001,), "f4"), ((2, 33 * 4096 + 5), "f4"), ((40003,), "f8")):
                dp.cumsum(dp.asarray(rng.normal(0, 1, shape).astype(dt)), axis=-1)
        finally:
            _lib.check(_lib.lib.dpb_set_tuning(b"scan_lookback_polls", -1))


def test_small_shape_sweeps_leave_the_guard_bytes_intact(guarded):
    import dpnp_b200 as dp

    lib, check = guarded
    for generic in (0, 1):
        check(lib.dpb_set_tuning(b"force_generic", generic))
        _sweep(dp)
        gc.collect()
        blocks, nbytes, first = _report(lib, check)
        assert (blocks, nbytes) == (0, 0), (generic, first)


def test_an_overrun_into_the_guard_zone_is_reported(guarded):
    lib, check = guarded
    from dpnp_b200 import _lib, get_default_queue

    q = get_default_queue()
    q.activate()
    p = C.c_void_p()
    check(lib.dpb_malloc(1000, C.c_void_p(q.stream), C.byref(p)))
    # 16 bytes past the block's end: still inside the allocation the library made (its guard zone)
    check(lib.dpb_memset(p, 0, 1016, C.c_void_p(q.stream)))
    check(lib.dpb_free(p, C.c_void_p(q.stream)))
    blocks, nbytes, first = _report(lib, check)
    assert blocks == 1 and nbytes == 16
    assert first[0] == p.value and first[1] == 1000 and 1000 <= first[2] < 1016
    assert _report(lib, check)[:2] == (0, 0)               # the report clears the counters
