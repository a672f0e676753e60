"""Callable objects behind every elementwise function.

``UnaryElementwiseFunc`` and ``BinaryElementwiseFunc`` carry the semantics of the
reference classes of the same name (dpnp/tensor/_elementwise_common.py:53-289 and
:292-988): execution placement, broadcasting, type promotion with cast buffers,
``out=`` validation and overlap handling, order-"K" result allocation and the
in-place operators.  The native calls they make are the functions of
``_tensor_elementwise_impl`` / ``_tensor_impl``.
"""

from __future__ import annotations

import numpy as np

from ..memory import ExecutionPlacementError
from . import _tensor_impl as ti
from ._copy_utils import (_empty, _empty_like_orderK, _empty_like_pair_orderK)
from ._ctors import asarray, empty_like
from ._manipulation_functions import _broadcast_shape_impl, broadcast_to
from ._type_utils import (_acceptance_fn_default_binary, _acceptance_fn_default_unary,
                          _find_buf_dtype, _find_buf_dtype2, _find_buf_dtype_in_place_op,
                          _get_dtype, _get_shape, _resolve_weak_types, _validate_dtype)
from .._lib import FLAG_C, FLAG_F
from ._usmarray import usm_ndarray


_scalar_cache: dict = {}


def _scalar_to_array(value, dtype, queue):
    """0-d device array holding a Python scalar.  The reference materialises every scalar
    operand with asarray() (dpnp/tensor/_elementwise_common.py:652-659), i.e. one host-to-
    device copy per call; here the arrays are kept per (queue, dtype, bit pattern) so that a
    repeated `x * 0.5` enqueues its kernel without touching the host-device link.  The
    cached arrays are only ever read."""
    dtype = np.dtype(dtype)
    try:
        bits = np.asarray(value).astype(dtype, casting="unsafe").tobytes()
    except (TypeError, ValueError, OverflowError):
        return asarray(value, dtype=dtype, sycl_queue=queue)
    key = (queue.device, queue.stream, dtype.char, bits)
    arr = _scalar_cache.get(key)
    if arr is None:
        if len(_scalar_cache) >= 4096:
            _scalar_cache.clear()
        arr = asarray(value, dtype=dtype, sycl_queue=queue)
        _scalar_cache[key] = arr
    return arr


_scalar_view_cache: dict = {}
_FLOATING = frozenset(np.dtype(c) for c in ("f2", "f4", "f8"))


def _scalar_operand(value, dtype, queue, shape):
    """The cached 0-d array of `_scalar_to_array` broadcast to `shape` (a stride-0 view), kept per
    (queue, type, value, shape) so that a repeated `x * 0.5` builds no Python objects at all."""
    key = (queue._stream, dtype.char, type(value), value.hex() if type(value) is float else value, shape)
    v = _scalar_view_cache.get(key)
    if v is None:
        if len(_scalar_view_cache) >= 4096:
            _scalar_view_cache.clear()
        v = _scalar_to_array(value, dtype, queue)
        if shape != ():
            v = broadcast_to(v, shape)
        _scalar_view_cache[key] = v
    return v


def _broadcast_operand(x, shape):
    """`x` broadcast to `shape` for a kernel call: the stride-0 view is remembered on the array
    (arrays are immutable in shape except through the `shape` setter, which drops the cache)."""
    cache = x._bcast_cache
    if cache is None:
        cache = x._bcast_cache = {}
    v = cache.get(shape)
    if v is None:
        if len(cache) >= 8:
            cache.clear()
        v = cache[shape] = broadcast_to(x, shape)
    return v


def _coerce_usm_type(types):
    """Result USM type: the first of device, shared, host that any input uses."""
    for t in ("device", "shared", "host"):
        if t in types:
            return t
    return "device"


def _common_queue(queues):
    """Queue shared by all inputs, or None if they live on different devices."""
    q0 = None
    for q in queues:
        if q is None:
            continue
        if q0 is None:
            q0 = q
        elif q.device != q0.device or q.stream != q0.stream:
            return None
    return q0


class UnaryElementwiseFunc:
    """out = f(x), elementwise."""

    def __init__(self, name, result_type_resolver_fn, unary_dp_impl_fn, docs,
                 acceptance_fn=_acceptance_fn_default_unary):
        self.__name__ = "UnaryElementwiseFunc"
        self.name_ = name
        self.result_type_resolver_fn_ = result_type_resolver_fn
        self.types_ = None
        self.unary_fn_ = unary_dp_impl_fn
        self.__doc__ = docs
        self.acceptance_fn_ = acceptance_fn
        self._direct_cache = {}

    def __str__(self):
        return f"<{self.__name__} '{self.name_}'>"

    __repr__ = __str__

    def get_implementation_function(self):
        return self.unary_fn_

    def get_type_result_resolver_function(self):
        return self.result_type_resolver_fn_

    def get_type_promotion_path_acceptance_function(self):
        return self.acceptance_fn_

    @property
    def nin(self):
        return 1

    @property
    def nout(self):
        return 1

    @property
    def types(self):
        """Supported signatures as 'in->out' character codes."""
        if self.types_ is None:
            from ._type_utils import _all_data_types
            self.types_ = []
            for dt in _all_data_types():
                r = self.result_type_resolver_fn_(dt)
                if r:
                    self.types_.append(f"{dt.char}->{r.char}")
        return self.types_

    def _direct(self, dt):
        """Result type when `dt` needs no cast buffer, else None (remembered per type)."""
        try:
            return self._direct_cache[dt]
        except KeyError:
            buf_dt, res_dt = _find_buf_dtype(dt, self.result_type_resolver_fn_, self.acceptance_fn_)
            r = self._direct_cache[dt] = res_dt if buf_dt is None else None
            return r

    def __call__(self, x, /, *, out=None, order="K"):
        if not isinstance(x, usm_ndarray):
            raise TypeError(f"Expected dpnp.tensor.usm_ndarray, got {type(x)}")
        if out is None and order == "K":
            # the common call: a dense input of a type the kernel takes as it is -- the general
            # path below computes exactly this (same result type, same layout), with more steps
            fl = x._flags
            res_dt = self._direct(x._dtype) if fl & (FLAG_C | FLAG_F) else None
            if res_dt is not None:
                q = x._queue
                out = usm_ndarray._new_dense(x._shape, res_dt, q, FLAG_C if fl & FLAG_C else FLAG_F, x._usm_type)
                self.unary_fn_(x, out, sycl_queue=q)
                return out
        if order not in ("C", "F", "K", "A"):
            order = "K"
        buf_dt, res_dt = _find_buf_dtype(x.dtype, self.result_type_resolver_fn_, self.acceptance_fn_)
        if res_dt is None:
            raise ValueError(
                f"function '{self.name_}' does not support input type ({x.dtype}), and the input "
                "could not be safely coerced to any supported types according to the casting rule "
                "''safe''.")
        exec_q = x.sycl_queue
        orig_out = out
        if out is not None:
            if not isinstance(out, usm_ndarray):
                raise TypeError(f"output array must be of usm_ndarray type, got {type(out)}")
            if not out.flags.writable:
                raise ValueError("provided `out` array is read-only")
            if out.shape != x.shape:
                raise ValueError("The shape of input and output arrays are inconsistent. "
                                 f"Expected output shape is {x.shape}, got {out.shape}")
            if res_dt != out.dtype:
                raise ValueError(f"Output array of type {res_dt} is needed, got {out.dtype}")
            if _common_queue((exec_q, out.sycl_queue)) is None:
                raise ExecutionPlacementError("Input and output allocation queues are not compatible")
            if buf_dt is None and ti._array_overlap(x, out) and not ti._same_logical_tensors(x, out):
                # partial overlap: compute into a temporary, copy back afterwards
                out = empty_like(out)
        if order == "A":
            order = "F" if (x.flags.f_contiguous and not x.flags.c_contiguous) else "C"
        src = x
        if buf_dt is not None:
            buf = _empty_like_orderK(x, buf_dt) if order == "K" else empty_like(x, dtype=buf_dt, order=order)
            ti._copy_usm_ndarray_into_usm_ndarray(x, buf, exec_q)
            src = buf
        if out is None:
            out = _empty_like_orderK(src, res_dt) if order == "K" else empty_like(src, dtype=res_dt, order=order)
        self.unary_fn_(src, out, sycl_queue=exec_q)
        if orig_out is not None and orig_out is not out:
            ti._copy_usm_ndarray_into_usm_ndarray(out, orig_out, exec_q)
            out = orig_out
        return out


class BinaryElementwiseFunc:
    """out = f(x1, x2), elementwise with broadcasting."""

    def __init__(self, name, result_type_resolver_fn, binary_dp_impl_fn, docs,
                 binary_inplace_fn=None, acceptance_fn=_acceptance_fn_default_binary,
                 weak_type_resolver=_resolve_weak_types):
        self.__name__ = "BinaryElementwiseFunc"
        self.name_ = name
        self.result_type_resolver_fn_ = result_type_resolver_fn
        self.types_ = None
        self.binary_fn_ = binary_dp_impl_fn
        self.binary_inplace_fn_ = binary_inplace_fn
        self.__doc__ = docs
        self.acceptance_fn_ = acceptance_fn
        self.weak_type_resolver_ = weak_type_resolver
        self._direct_cache = {}
        self._promo_cache = {}

    def __str__(self):
        return f"<{self.__name__} '{self.name_}'>"

    __repr__ = __str__

    def get_type_result_resolver_function(self):
        return self.result_type_resolver_fn_

    def get_implementation_function(self):
        return self.binary_fn_

    def get_implementation_inplace_function(self):
        return self.binary_inplace_fn_

    def get_type_promotion_path_acceptance_function(self):
        return self.acceptance_fn_

    def get_array_dtype_scalar_type_resolver_function(self):
        return self.weak_type_resolver_

    @property
    def nin(self):
        return 2

    @property
    def nout(self):
        return 1

    @property
    def types(self):
        if self.types_ is None:
            from ._type_utils import _all_data_types
            self.types_ = []
            for d1 in _all_data_types():
                for d2 in _all_data_types():
                    r = self.result_type_resolver_fn_(d1, d2)
                    if r:
                        self.types_.append(f"{d1.char}{d2.char}->{r.char}")
        return self.types_

    # ---------------------------------------------------------------- helpers
    @staticmethod
    def _placement(o1, o2):
        q1 = o1.sycl_queue if isinstance(o1, usm_ndarray) else None
        q2 = o2.sycl_queue if isinstance(o2, usm_ndarray) else None
        if q1 is None and q2 is None:
            raise ExecutionPlacementError(
                "Execution placement can not be unambiguously inferred from input arguments. "
                "One of the arguments must represent USM allocation and expose "
                "`__sycl_usm_array_interface__` property")
        exec_q = _common_queue((q1, q2))
        if exec_q is None:
            raise ExecutionPlacementError(
                "Execution placement can not be unambiguously inferred from input arguments.")
        types = [o.usm_type for o in (o1, o2) if isinstance(o, usm_ndarray)]
        return exec_q, _coerce_usm_type(types)

    def _resolve(self, o1, o2):
        o1_shape, o2_shape = _get_shape(o1), _get_shape(o2)
        if not all(isinstance(s, (tuple, list)) for s in (o1_shape, o2_shape)):
            raise TypeError("Shape of arguments can not be inferred. Arguments are expected to be "
                            "lists, tuples, or both")
        try:
            res_shape = _broadcast_shape_impl([o1_shape, o2_shape])
        except ValueError:
            raise ValueError("operands could not be broadcast together with shapes "
                             f"{o1_shape} and {o2_shape}") from None
        o1_dtype, o2_dtype = _get_dtype(o1), _get_dtype(o2)
        if not all(_validate_dtype(o) for o in (o1_dtype, o2_dtype)):
            raise ValueError("Operands have unsupported data types")
        o1_dtype, o2_dtype = self.weak_type_resolver_(o1_dtype, o2_dtype, None)
        return res_shape, o1_dtype, o2_dtype

    # ------------------------------------------------------------------- call
    def _direct(self, dt):
        """Result type for two operands of type `dt` when neither needs a cast buffer, else None."""
        try:
            return self._direct_cache[dt]
        except KeyError:
            b1, b2, res_dt = _find_buf_dtype2(dt, dt, self.result_type_resolver_fn_, self.acceptance_fn_)
            r = self._direct_cache[dt] = res_dt if (b1 is None and b2 is None) else None
            return r

    def __call__(self, o1, o2, /, *, out=None, order="K"):
        if out is None and order == "K" and type(o1) is usm_ndarray and type(o2) is usm_ndarray:
            # the common call: two arrays of one type and shape on one queue, at least one of them
            # dense -- the general path below computes exactly this (same result type; order "K"
            # gives C order when either input is C-contiguous, F order when both are F-contiguous)
            f1, f2 = o1._flags, o2._flags
            if (o1._shape == o2._shape and o1._queue is o2._queue and o1._dtype == o2._dtype
                    and o1._usm_type == o2._usm_type):
                order_flag = FLAG_C if (f1 | f2) & FLAG_C else (FLAG_F if f1 & f2 & FLAG_F else 0)
                res_dt = self._direct(o1._dtype) if order_flag else None
                if res_dt is not None:
                    q = o1._queue
                    out = usm_ndarray._new_dense(o1._shape, res_dt, q, order_flag, o1._usm_type)
                    self.binary_fn_(o1, o2, out, sycl_queue=q)
                    return out
        elif out is None and order == "K":
            # a dense floating array and a Python float or int: the scalar takes the array's type
            # (NEP 50, `_promote_weak`), so this is the case above with a stride-0 second operand
            t1, t2 = type(o1), type(o2)
            if t1 is usm_ndarray and (t2 is float or t2 is int):
                arr, sc, first = o1, o2, True
            elif t2 is usm_ndarray and (t1 is float or t1 is int):
                arr, sc, first = o2, o1, False
            else:
                arr = None
            if arr is not None and arr._dtype in _FLOATING and arr._flags & (FLAG_C | FLAG_F):
                dt = arr._dtype
                res_dt = self._direct(dt)
                if res_dt is not None:
                    q = arr._queue
                    view = _scalar_operand(sc, dt, q, arr._shape)
                    out = usm_ndarray._new_dense(arr._shape, res_dt, q,
                                                 FLAG_C if arr._flags & FLAG_C else FLAG_F, arr._usm_type)
                    if first:
                        self.binary_fn_(arr, view, out, sycl_queue=q)
                    else:
                        self.binary_fn_(view, arr, out, sycl_queue=q)
                    return out
        if order not in ("K", "C", "F", "A"):
            order = "K"
        if type(o1) is usm_ndarray and type(o2) is usm_ndarray:
            # two arrays: placement, broadcast shape and promotion without the scalar handling
            q1, q2 = o1._queue, o2._queue
            if not (q1 is q2 or (q1.device == q2.device and q1._stream == q2._stream)):
                raise ExecutionPlacementError(
                    "Execution placement can not be unambiguously inferred from input arguments.")
            exec_q = q1
            res_usm_type = o1._usm_type if o1._usm_type == o2._usm_type else _coerce_usm_type(
                (o1._usm_type, o2._usm_type))
            if o1._shape == o2._shape:
                res_shape = o1._shape
            else:
                try:
                    res_shape = _broadcast_shape_impl([o1._shape, o2._shape])
                except ValueError:
                    raise ValueError("operands could not be broadcast together with shapes "
                                     f"{o1._shape} and {o2._shape}") from None
            o1_dtype, o2_dtype = o1._dtype, o2._dtype
            try:
                buf1_dt, buf2_dt, res_dt = self._promo_cache[(o1_dtype, o2_dtype)]
            except KeyError:
                buf1_dt, buf2_dt, res_dt = self._promo_cache[(o1_dtype, o2_dtype)] = _find_buf_dtype2(
                    o1_dtype, o2_dtype, self.result_type_resolver_fn_, self.acceptance_fn_)
        else:
            exec_q, res_usm_type = self._placement(o1, o2)
            res_shape, o1_dtype, o2_dtype = self._resolve(o1, o2)
            buf1_dt, buf2_dt, res_dt = _find_buf_dtype2(o1_dtype, o2_dtype, self.result_type_resolver_fn_,
                                                        self.acceptance_fn_)
        if res_dt is None:
            raise ValueError(
                f"function '{self.name_}' does not support input types ({o1_dtype}, {o2_dtype}), "
                "and the inputs could not be safely coerced to any supported types according to "
                "the casting rule ''safe''.")
        orig_out = out
        if out is not None:
            if not isinstance(out, usm_ndarray):
                raise TypeError(f"output array must be of usm_ndarray type, got {type(out)}")
            if not out.flags.writable:
                raise ValueError("provided `out` array is read-only")
            if out.shape != res_shape:
                raise ValueError("The shape of input and output arrays are inconsistent. "
                                 f"Expected output shape is {res_shape}, got {out.shape}")
            if res_dt != out.dtype:
                raise ValueError(f"Output array of type {res_dt} is needed, got {out.dtype}")
            if _common_queue((exec_q, out.sycl_queue)) is None:
                raise ExecutionPlacementError("Input and output allocation queues are not compatible")
            if isinstance(o1, usm_ndarray) and buf1_dt is None and ti._array_overlap(o1, out):
                if not ti._same_logical_tensors(o1, out):
                    out = empty_like(out)
                elif self.binary_inplace_fn_ is not None:
                    # `out` is `o1`: use the in-place kernel
                    if isinstance(o2, usm_ndarray):
                        src2 = o2
                        if (buf2_dt is None and ti._array_overlap(o2, out)
                                and not ti._same_logical_tensors(o2, out)):
                            buf2_dt = o2_dtype
                    else:
                        src2 = _scalar_to_array(o2, o2_dtype, exec_q)
                    if buf2_dt is not None:
                        buf2 = empty_like(src2, dtype=buf2_dt)
                        ti._copy_usm_ndarray_into_usm_ndarray(src2, buf2, exec_q)
                        src2 = buf2
                    if src2.shape != res_shape:
                        src2 = broadcast_to(src2, res_shape)
                    self.binary_inplace_fn_(o1, src2, sycl_queue=exec_q)
                    return out
            if (isinstance(o2, usm_ndarray) and buf2_dt is None and out is orig_out
                    and ti._array_overlap(o2, out) and not ti._same_logical_tensors(o2, out)):
                out = empty_like(out)

        src1 = o1 if isinstance(o1, usm_ndarray) else _scalar_to_array(o1, o1_dtype, exec_q)
        src2 = o2 if isinstance(o2, usm_ndarray) else _scalar_to_array(o2, o2_dtype, exec_q)
        if order == "A":
            order = "F" if all(a.flags.f_contiguous for a in (src1, src2)) else "C"

        # cast buffers where promotion asks for them
        if buf1_dt is not None:
            b = _empty_like_orderK(src1, buf1_dt) if order == "K" else empty_like(src1, dtype=buf1_dt, order=order)
            ti._copy_usm_ndarray_into_usm_ndarray(src1, b, exec_q)
            src1 = b
        if buf2_dt is not None:
            b = _empty_like_orderK(src2, buf2_dt) if order == "K" else empty_like(src2, dtype=buf2_dt, order=order)
            ti._copy_usm_ndarray_into_usm_ndarray(src2, b, exec_q)
            src2 = b
        if out is None:
            if order == "K":
                out = _empty_like_pair_orderK(src1, src2, res_dt, res_shape, res_usm_type, exec_q)
            else:
                out = _empty(res_shape, res_dt, exec_q, order, res_usm_type)
        if src1._shape != res_shape:
            src1 = _broadcast_operand(src1, res_shape)
        if src2._shape != res_shape:
            src2 = _broadcast_operand(src2, res_shape)
        self.binary_fn_(src1, src2, out, sycl_queue=exec_q)
        if orig_out is not None and orig_out is not out:
            ti._copy_usm_ndarray_into_usm_ndarray(out, orig_out, exec_q)
            out = orig_out
        return out

    # --------------------------------------------------------------- in place
    def _inplace_op(self, o1, o2):
        """o1 <op>= o2 (dpnp/tensor/_elementwise_common.py:853-988)."""
        if self.binary_inplace_fn_ is None:
            raise ValueError("binary function does not have a dedicated in-place implementation")
        if not isinstance(o1, usm_ndarray):
            raise TypeError(f"Left-hand side argument must be of usm_ndarray type, got {type(o1)}")
        if not o1.flags.writable:
            raise ValueError("provided left-hand side array is read-only")
        q2 = o2.sycl_queue if isinstance(o2, usm_ndarray) else None
        exec_q = _common_queue((o1.sycl_queue, q2))
        if exec_q is None:
            raise ExecutionPlacementError(
                "Execution placement can not be unambiguously inferred from input arguments.")
        o1_shape, o2_shape = o1.shape, _get_shape(o2)
        if not isinstance(o2_shape, (tuple, list)):
            raise TypeError("Shape of second argument can not be inferred. Expected list or tuple.")
        try:
            res_shape = _broadcast_shape_impl([o1_shape, o2_shape])
        except ValueError:
            raise ValueError("operands could not be broadcast together with shapes "
                             f"{o1_shape} and {o2_shape}") from None
        if res_shape != o1_shape:
            raise ValueError(f"The shape of the non-broadcastable left-hand side {o1_shape} is "
                             f"inconsistent with the broadcast shape {res_shape}.")
        o1_dtype, o2_dtype = o1.dtype, _get_dtype(o2)
        if not _validate_dtype(o2_dtype):
            raise ValueError("Operand has an unsupported data type")
        o1_dtype, o2_dtype = self.weak_type_resolver_(o1_dtype, o2_dtype, None)
        buf_dt, res_dt = _find_buf_dtype_in_place_op(o1_dtype, o2_dtype, self.result_type_resolver_fn_)
        if res_dt is None:
            raise ValueError(
                f"function '{self.name_}' does not support input types ({o1_dtype}, {o2_dtype}), "
                "and the inputs could not be safely coerced to any supported types according to "
                "the casting rule ''same_kind''.")
        if res_dt != o1_dtype:
            raise ValueError(f"Output array of type {res_dt} is needed, got {o1_dtype}")
        if isinstance(o2, usm_ndarray):
            src2 = o2
            if (buf_dt is None and ti._array_overlap(o2, o1) and not ti._same_logical_tensors(o2, o1)):
                buf_dt = o2_dtype
        else:
            src2 = _scalar_to_array(o2, o2_dtype, exec_q)
        if buf_dt is not None:
            buf = empty_like(src2, dtype=buf_dt)
            ti._copy_usm_ndarray_into_usm_ndarray(src2, buf, exec_q)
            src2 = buf
        if src2.shape != res_shape:
            src2 = broadcast_to(src2, res_shape)
        self.binary_inplace_fn_(o1, src2, sycl_queue=exec_q)
        return o1
