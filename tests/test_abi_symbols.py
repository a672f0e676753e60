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
