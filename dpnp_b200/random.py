"""Device-side random fills.

The reference draws with oneMKL engines on the device
(dpnp/random/dpnp_iface_random.py:1663,1965-2033; dpnp/random/dpnp_random_state.py:84-116);
its streams cannot be reproduced elsewhere, so parity is never checked on
random output.  Here a counter-based generator fills arrays directly in device
memory: element i depends only on (seed, call counter, i).
"""

from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from ._lib import check, lib
from .dpnp_array import dpnp_array
from .memory import normalize_queue
from .tensor._copy_utils import _empty

_state = {"seed": 0x5EED, "calls": 0}


def seed(seed=None):
    _state["seed"] = 0x5EED if seed is None else int(seed) & 0xFFFFFFFFFFFFFFFF
    _state["calls"] = 0


def _next_seed():
    s = (_state["seed"] * 0x9E3779B97F4A7C15 + _state["calls"] * 0xD1B54A32D192ED03 + 1) & 0xFFFFFFFFFFFFFFFF
    _state["calls"] += 1
    return s


def _shape(size):
    if size is None:
        return ()
    return (int(size),) if isinstance(size, (int, np.integer)) else tuple(int(s) for s in size)


def uniform(low=0.0, high=1.0, size=None, device=None, usm_type="device", sycl_queue=None, dtype=None):
    """Samples from U[low, high)."""
    q = normalize_queue(sycl_queue, device)
    dt = np.dtype("f8") if dtype is None else np.dtype(dtype)
    res = _empty(_shape(size), dt, q, "C", usm_type)
    if res.size:
        q.activate()
        check(lib.dpb_random_uniform(_lib.typenum_of(dt), C.c_void_p(res._ptr), res.size, float(low),
                                     float(high), _next_seed(), 0, C.c_void_p(q.stream)))
    return dpnp_array._create_from_usm_ndarray(res)


def random(size=None, device=None, usm_type="device", sycl_queue=None):
    return uniform(0.0, 1.0, size, device=device, usm_type=usm_type, sycl_queue=sycl_queue)


rand = lambda *shape, **kw: uniform(0.0, 1.0, shape, **kw)  # noqa: E731


def normal(loc=0.0, scale=1.0, size=None, device=None, usm_type="device", sycl_queue=None, dtype=None):
    """Samples from N(loc, scale^2)."""
    q = normalize_queue(sycl_queue, device)
    dt = np.dtype("f8") if dtype is None else np.dtype(dtype)
    res = _empty(_shape(size), dt, q, "C", usm_type)
    if res.size:
        q.activate()
        check(lib.dpb_random_normal(_lib.typenum_of(dt), C.c_void_p(res._ptr), res.size, float(loc),
                                    float(scale), _next_seed(), 0, C.c_void_p(q.stream)))
    return dpnp_array._create_from_usm_ndarray(res)


def randn(*shape, **kw):
    return normal(0.0, 1.0, shape, **kw)


def randint(low, high=None, size=None, dtype=int, device=None, usm_type="device", sycl_queue=None):
    """Integers uniformly distributed in [low, high)."""
    if high is None:
        low, high = 0, low
    q = normalize_queue(sycl_queue, device)
    dt = np.dtype("i8") if dtype is int else np.dtype(dtype)
    res = _empty(_shape(size), dt, q, "C", usm_type)
    if res.size:
        q.activate()
        check(lib.dpb_random_uniform(_lib.typenum_of(dt), C.c_void_p(res._ptr), res.size, float(low),
                                     float(high), _next_seed(), 0, C.c_void_p(q.stream)))
    return dpnp_array._create_from_usm_ndarray(res)
