"""The C-ABI library loads without a GPU and exports every symbol the header declares."""

import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "dpnp_b200.h")


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(dpb_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_symbols():
    syms = declared_symbols()
    assert len(syms) > 50
    assert "dpb_binary_ufunc" in syms and "dpb_reduction_over_axis" in syms


def test_library_exports_every_declared_symbol():
    from dpnp_b200 import _lib

    lib = ctypes.CDLL(_lib.LIB_PATH)
    missing = [s for s in declared_symbols() if not hasattr(lib, s)]
    assert not missing, f"symbols declared in the header but not exported: {missing}"


def test_python_prototypes_cover_the_header():
    from dpnp_b200 import _lib

    assert sorted(_lib.PROTOTYPES) == declared_symbols()


def test_version_and_error_channel():
    from dpnp_b200 import _lib

    assert b"sm_100a" in _lib.lib.dpb_version()
    st = _lib.lib.dpb_set_tuning(b"no_such_key", 1)
    assert st == _lib.ERR_VALUE
    assert "unknown tuning key" in _lib.last_error()
    with pytest.raises(ValueError):
        _lib.check(st)


def test_result_type_tables_need_no_device():
    from dpnp_b200 import _lib

    f4 = _lib.typenum_of("f4")
    assert _lib.lib.dpb_binary_result_type(_lib.BINARY_OPS["add"], f4, f4) == f4
    assert _lib.lib.dpb_binary_result_type(_lib.BINARY_OPS["less"], f4, f4) == _lib.typenum_of("?")
    # subtract has no boolean form; exp has no integer form; erf(f16) -> f32
    b = _lib.typenum_of("?")
    assert _lib.lib.dpb_binary_result_type(_lib.BINARY_OPS["subtract"], b, b) == -1
    assert _lib.lib.dpb_unary_result_type(_lib.UNARY_OPS["exp"], _lib.typenum_of("i4")) == -1
    assert _lib.lib.dpb_unary_result_type(_lib.UNARY_OPS["erf"], _lib.typenum_of("f2")) == f4
    # mixed signed/unsigned 64-bit comparisons exist, mixed add does not
    i8, u8 = _lib.typenum_of("i8"), _lib.typenum_of("u8")
    assert _lib.lib.dpb_binary_result_type(_lib.BINARY_OPS["less"], i8, u8) == b
    assert _lib.lib.dpb_binary_result_type(_lib.BINARY_OPS["add"], i8, u8) == -1
    assert _lib.lib.dpb_reduce_dtype_supported(_lib.REDUCE_OPS["sum"], _lib.typenum_of("i4"), i8) == 1
    assert _lib.lib.dpb_reduce_dtype_supported(_lib.REDUCE_OPS["sum"], f4, _lib.typenum_of("i4")) == 0


def test_pool_limit_fails_before_touching_a_device():
    from dpnp_b200 import _lib

    _lib.check(_lib.lib.dpb_pool_set_limit(1024))
    try:
        p = ctypes.c_void_p()
        st = _lib.lib.dpb_malloc(4096, None, ctypes.byref(p))
        assert st == _lib.ERR_MEMORY
        with pytest.raises(MemoryError):
            _lib.check(st)
    finally:
        _lib.check(_lib.lib.dpb_pool_set_limit(0))


def test_compute_entry_points_fail_loudly_without_a_device():
    from dpnp_b200 import _lib

    if _lib.device_count() > 0:
        pytest.skip("a device is present")
    import dpnp_b200 as dp

    with pytest.raises(RuntimeError):
        dp.zeros(4)


def test_runtime_switches_are_settable_without_a_device():
    from dpnp_b200 import _lib

    lib = _lib.lib
    for key in (b"verbose", b"force_generic"):
        assert lib.dpb_set_tuning(key, 1) == _lib.OK
        assert lib.dpb_set_tuning(key, 0) == _lib.OK
        assert lib.dpb_set_tuning(key, 2) == _lib.ERR_VALUE
    assert lib.dpb_set_tuning(b"no_such_switch", 1) == _lib.ERR_VALUE
    assert "no_such_switch" in _lib.last_error()


def test_the_pybind11_shim_is_built_and_bound_to_the_same_library():
    from dpnp_b200 import _lib

    assert _lib.native is not None, "dpnp_b200/_tensor_native*.so is missing: run python dpnp_b200/_build.py"
    assert _lib.native.version() == _lib.lib.dpb_version().decode()
    core = _lib.native.ArrayCore(4096, _lib.typenum_of("f4"), 7, 0, (3, 5), (5, 1))
    assert (core.ptr, core.typenum, core.flags, core.device) == (4096, 10, 7, 0)
    with pytest.raises(ValueError):
        _lib.native.ArrayCore(0, 10, 7, 0, (3, 5), (1,))
    # status codes of the library arrive as the exceptions the reference's modules raise
    a = _lib.native.ArrayCore(0, 10, 7, 0, (4,), (1,))
    b = _lib.native.ArrayCore(0, 10, 7, 0, (5,), (1,))
    with pytest.raises((ValueError, RuntimeError)):
        _lib.native.binary(0, a, a, b, 0)
