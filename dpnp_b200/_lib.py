"""ctypes binding of libdpnp_b200.so (the C ABI declared in include/dpnp_b200.h).

The library is the product: if it cannot be loaded, importing the compute
layers fails loudly -- there is no CPU fallback.  Status codes are mapped to
the exception classes the reference's pybind11 dispatchers raise
(``ValueError`` for ``py::value_error``, ``RuntimeError`` for
``std::runtime_error``; dpnp/tensor/libtensor/source/elementwise_functions/
elementwise_functions.hpp:96-164).
"""

from __future__ import annotations

import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libdpnp_b200.so")

MAX_ND = 32

# typenum ids, same order as the C enum dpb_typenum
_DTYPES = [
    np.dtype("?"), np.dtype("i1"), np.dtype("u1"), np.dtype("i2"), np.dtype("u2"),
    np.dtype("i4"), np.dtype("u4"), np.dtype("i8"), np.dtype("u8"),
    np.dtype("f2"), np.dtype("f4"), np.dtype("f8"), np.dtype("c8"), np.dtype("c16"),
]
_TYPENUM = {dt: i for i, dt in enumerate(_DTYPES)}


def typenum_of(dtype) -> int:
    """Type id of a NumPy dtype; raises TypeError for unsupported dtypes."""
    dt = np.dtype(dtype)
    try:
        return _TYPENUM[dt]
    except KeyError:
        raise TypeError(f"data type {dt} is not supported") from None


def dtype_of(typenum: int) -> np.dtype:
    return _DTYPES[typenum]


def supported_dtypes():
    return list(_DTYPES)


# unary / binary / reduction op ids (dpb_unary_op, dpb_binary_op, ... in the header)
UNARY_OPS = {name: i for i, name in enumerate([
    "negative", "positive", "abs", "exp", "log", "sqrt", "erf", "square", "reciprocal",
    "sin", "cos", "tanh", "expm1", "log1p", "floor", "ceil", "sign", "logical_not",
    "isnan", "isfinite", "isinf", "acos", "acosh", "asin", "asinh", "atan", "atanh", "cbrt", "cosh", "sinh",
    "tan", "exp2", "log2", "log10", "rsqrt", "trunc", "round", "signbit", "bitwise_invert", "conj", "real",
    "imag", "angle", "proj"])}
BINARY_OPS = {name: i for i, name in enumerate([
    "add", "subtract", "multiply", "divide", "maximum", "minimum", "equal", "not_equal",
    "less", "less_equal", "greater", "greater_equal", "logical_and", "logical_or", "pow", "atan2", "hypot",
    "copysign", "logaddexp", "nextafter", "bitwise_and", "bitwise_or", "bitwise_xor", "bitwise_left_shift",
    "bitwise_right_shift", "floor_divide", "remainder", "logical_xor"])}
REDUCE_OPS = {"sum": 0, "prod": 1, "max": 2, "min": 3, "logsumexp": 4, "hypot": 5}
SEARCH_OPS = {"argmax": 0, "argmin": 1}
ACCUMULATE_OPS = {"cumsum": 0, "cumprod": 1, "cumlogsumexp": 2}

OK, ERR_VALUE, ERR_RUNTIME, ERR_CUDA, ERR_MEMORY, ERR_TYPE = range(6)

FLAG_C, FLAG_F, FLAG_W = 1, 2, 4


class dpb_array(C.Structure):
    _fields_ = [
        ("data", C.c_void_p),
        ("nd", C.c_int32),
        ("typenum", C.c_int32),
        ("flags", C.c_int32),
        ("device", C.c_int32),
        ("shape", C.POINTER(C.c_int64)),
        ("strides", C.POINTER(C.c_int64)),
    ]


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python dpnp_b200/_build.py` "
            "(there is no CPU fallback)"
        )
    return C.CDLL(LIB_PATH)


lib = _load()

_vp, _i, _i64, _sz, _dbl, _u64 = C.c_void_p, C.c_int, C.c_int64, C.c_size_t, C.c_double, C.c_uint64
_pvp = C.POINTER(C.c_void_p)
_pi64 = C.POINTER(C.c_int64)
_parr = C.POINTER(dpb_array)

# name -> (restype, argtypes).  Every symbol the header declares is listed.
PROTOTYPES = {
    "dpb_last_error": (C.c_char_p, []),
    "dpb_version": (C.c_char_p, []),
    "dpb_device_count": (_i, []),
    "dpb_set_device": (_i, [_i]),
    "dpb_get_device": (_i, [C.POINTER(_i)]),
    "dpb_device_info": (_i, [_i, C.POINTER(_i), C.POINTER(_sz), C.POINTER(_i), C.POINTER(_i)]),
    "dpb_stream_create": (_i, [_pvp]),
    "dpb_stream_destroy": (_i, [_vp]),
    "dpb_stream_synchronize": (_i, [_vp]),
    "dpb_device_synchronize": (_i, []),
    "dpb_event_create": (_i, [_pvp]),
    "dpb_event_destroy": (_i, [_vp]),
    "dpb_event_record": (_i, [_vp, _vp]),
    "dpb_event_synchronize": (_i, [_vp]),
    "dpb_stream_wait_event": (_i, [_vp, _vp]),
    "dpb_event_elapsed_ms": (_i, [_vp, _vp, C.POINTER(C.c_float)]),
    "dpb_malloc": (_i, [_sz, _vp, _pvp]),
    "dpb_free": (_i, [_vp, _vp]),
    "dpb_pool_trim": (_i, [_sz]),
    "dpb_debug_redzone_report": (_i, [_pi64, _pi64, _pi64]),
    "dpb_pool_stats": (_i, [C.POINTER(_sz)] * 4),
    "dpb_pool_set_limit": (_i, [_sz]),
    "dpb_host_alloc": (_i, [_sz, _pvp]),
    "dpb_host_free": (_i, [_vp]),
    "dpb_memcpy": (_i, [_vp, _vp, _sz, _i, _vp]),
    "dpb_memset": (_i, [_vp, _i, _sz, _vp]),
    "dpb_simplify_iteration_space": (_i, [_i, _i, _pi64, _pi64, _pi64, C.POINTER(_i)]),
    "dpb_compact_iteration": (_i, [_i, _pi64, _pi64, C.POINTER(_i)]),
    "dpb_array_overlap": (_i, [_parr, _parr, C.POINTER(_i)]),
    "dpb_same_logical_tensors": (_i, [_parr, _parr, C.POINTER(_i)]),
    "dpb_unary_contig": (_i, [_i, _i, _i, _i64, _vp, _i64, _vp, _i64, _vp]),
    "dpb_unary_strided": (_i, [_i, _i, _i, _i64, _i, _pi64, _vp, _i64, _vp, _i64, _vp]),
    "dpb_binary_contig": (_i, [_i, _i, _i, _i, _i64, _vp, _i64, _vp, _i64, _vp, _i64, _vp]),
    "dpb_binary_strided": (_i, [_i, _i, _i, _i, _i64, _i, _pi64, _vp, _i64, _vp, _i64, _vp, _i64, _vp]),
    "dpb_binary_inplace_contig": (_i, [_i, _i, _i, _i64, _vp, _i64, _vp, _i64, _vp]),
    "dpb_binary_inplace_strided": (_i, [_i, _i, _i, _i64, _i, _pi64, _vp, _i64, _vp, _i64, _vp]),
    "dpb_where_contig": (_i, [_i, _i, _i64, _vp, _vp, _vp, _vp, _vp]),
    "dpb_where_strided": (_i, [_i, _i, _i64, _i, _pi64, _vp, _i64, _vp, _i64, _vp, _i64, _vp, _i64, _vp]),
    "dpb_copy_cast_contig": (_i, [_i, _i, _i64, _vp, _i64, _vp, _i64, _vp]),
    "dpb_copy_cast_strided": (_i, [_i, _i, _i64, _i, _pi64, _vp, _i64, _vp, _i64, _vp]),
    "dpb_reduce_axis1_contig": (_i, [_i, _i, _i, _i64, _i64, _vp, _i64, _vp, _i64, _vp]),
    "dpb_reduce_axis0_contig": (_i, [_i, _i, _i, _i64, _i64, _vp, _i64, _vp, _i64, _vp]),
    "dpb_reduce_axis1_contig_noalloc": (_i, [_i, _i, _i, _i64, _i64, _vp, _i64, _vp, _i64, _vp]),
    "dpb_reduce_strided": (_i, [_i, _i, _i, _i64, _i64, _vp, _vp, _i, _pi64, _i64, _i64, _i, _pi64, _i64, _vp]),
    "dpb_search_axis1_contig": (_i, [_i, _i, _i64, _i64, _vp, _i64, _vp, _i64, _vp]),
    "dpb_search_axis0_contig": (_i, [_i, _i, _i64, _i64, _vp, _i64, _vp, _i64, _vp]),
    "dpb_search_strided": (_i, [_i, _i, _i64, _i64, _vp, _vp, _i, _pi64, _i64, _i64, _i, _pi64, _i64, _vp]),
    "dpb_unary_result_type": (_i, [_i, _i]),
    "dpb_binary_result_type": (_i, [_i, _i, _i]),
    "dpb_unary_ufunc": (_i, [_i, _parr, _parr, _vp]),
    "dpb_binary_ufunc": (_i, [_i, _parr, _parr, _parr, _vp]),
    "dpb_binary_inplace_ufunc": (_i, [_i, _parr, _parr, _vp]),
    "dpb_where": (_i, [_parr, _parr, _parr, _parr, _vp]),
    "dpb_copy_array_into_array": (_i, [_parr, _parr, _vp]),
    "dpb_divide_by_scalar": (_i, [_parr, _dbl, _parr, _vp]),
    "dpb_full_array": (_i, [_parr, _vp, _vp]),
    "dpb_reduce_dtype_supported": (_i, [_i, _i, _i]),
    "dpb_reduction_over_axis": (_i, [_i, _parr, _i, _parr, _vp]),
    "dpb_search_over_axis": (_i, [_i, _parr, _i, _parr, _vp]),
    "dpb_black_scholes_f64": (_i, [_i64, _vp, _vp, _vp, _dbl, _dbl, _vp, _vp, _vp]),
    "dpb_fused_elementwise": (_i, [_vp, _i64, _vp]),
    "dpb_fused_elementwise_specialized": (_i, [_vp, _i64, _vp]),
    "dpb_fused_specialize_available": (_i, []),
    "dpb_fused_set_include_path": (_i, [C.c_char_p]),
    "dpb_fused_specialized_source": (_i, [_vp, C.c_char_p, _i64, _pi64]),
    "dpb_fused_specialize_compile": (_i, [_vp, _pi64]),
    "dpb_accumulate_over_axis": (_i, [_i, _parr, _parr, _i, _vp]),
    "dpb_accumulate_dtype_supported": (_i, [_i, _i, _i]),
    "dpb_random_uniform": (_i, [_i, _vp, _i64, _dbl, _dbl, _u64, _u64, _vp]),
    "dpb_random_normal": (_i, [_i, _vp, _i64, _dbl, _dbl, _u64, _u64, _vp]),
    "dpb_linspace_step": (_i, [_i, _vp, _i64, _vp, _vp, _vp]),
    "dpb_linspace_affine": (_i, [_i, _vp, _i64, _vp, _vp, _i, _vp]),
    "dpb_take_one": (_i, [_i, _vp, _i64, _vp, _vp, _vp]),
    "dpb_probe_fp64_fma": (_i, [_i64, _i, _vp, _i64, _pi64, _vp]),
    "dpb_comm_load": (_i, [C.c_char_p]),
    "dpb_comm_nccl_version": (_i, [C.POINTER(_i)]),
    "dpb_comm_unique_id": (_i, [_vp]),
    "dpb_comm_init": (_i, [_i, _i, _vp, _pvp]),
    "dpb_device_pci_bus_id": (_i, [_i, C.c_char_p, _i]),
    "dpb_comm_peer_export": (_i, [_vp, _vp, _i64, _pi64]),
    "dpb_comm_peer_attach": (_i, [_vp, _vp, _i]),
    "dpb_comm_peer_enable": (_i, [_vp, _i]),
    "dpb_comm_peer_probe_wait": (_i, [_vp, _i64, C.POINTER(_i), _vp]),
    "dpb_comm_destroy": (_i, [_vp]),
    "dpb_comm_info": (_i, [_vp, C.POINTER(_i), C.POINTER(_i)]),
    "dpb_comm_allgather": (_i, [_vp, _vp, _vp, _i64, _vp]),
    "dpb_comm_sum_ordered": (_i, [_vp, _i, _vp, _vp, _i64, _vp]),
    "dpb_comm_extreme": (_i, [_vp, _i, _i, _vp, _vp, _i64, _vp]),
    "dpb_comm_arg_extreme": (_i, [_vp, _i, _i, _vp, _i64, _vp, _i64, _vp, _vp, _vp]),
    "dpb_last_kernel": (C.c_char_p, []),
    "dpb_launch_count": (_i64, []),
    "dpb_reset_launch_count": (None, []),
    "dpb_set_tuning": (_i, [C.c_char_p, _i64]),
}

for _name, (_res, _args) in PROTOTYPES.items():
    try:
        _fn = getattr(lib, _name)
    except AttributeError:
        raise ImportError(f"{LIB_PATH} does not export {_name}: it is older than the sources, rebuild it "
                          "with `python dpnp_b200/_build.py`") from None
    _fn.restype = _res
    _fn.argtypes = _args


# The pybind11 shim (csrc/pyshim/tensor_native.cpp) is the binding the hot calls go through: it
# hands the library a `dpb_array` kept on each Python array and costs about a microsecond per
# call.  ctypes above stays the binding of everything else, and of the hot calls too when the
# shim has not been built (`native is None`); both reach the same library and the same kernels.
try:
    from . import _tensor_native as native
except ImportError:
    if os.environ.get("DPNP_B200_REQUIRE_NATIVE"):
        raise
    native = None


def last_error() -> str:
    return lib.dpb_last_error().decode("utf-8", "replace")


def check(status: int) -> None:
    """Raise the exception matching a non-zero dpb_status."""
    if status == OK:
        return
    msg = last_error()
    if status == ERR_VALUE:
        raise ValueError(msg)
    if status == ERR_MEMORY:
        raise MemoryError(msg)
    if status == ERR_TYPE:
        raise TypeError(msg)
    raise RuntimeError(msg)


def device_count() -> int:
    return int(lib.dpb_device_count())


def last_kernel() -> str:
    return lib.dpb_last_kernel().decode()


def launch_count() -> int:
    return int(lib.dpb_launch_count())


def reset_launch_count() -> None:
    lib.dpb_reset_launch_count()
