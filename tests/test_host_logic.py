"""Host-side semantics that need no device: type promotion, broadcasting, basic
slicing, reshape strides, contiguity flags, order-K permutation."""

import numpy as np
import pytest

from dpnp_b200.tensor import _elementwise_funcs as ef
from dpnp_b200.tensor import _type_utils as tu
from dpnp_b200.tensor._manipulation_functions import _broadcast_shape_impl, _reshape_strides
from dpnp_b200.tensor._slicing import basic_slice_meta
from dpnp_b200.tensor._usmarray import _contig_flags

ALL = tu._all_data_types()
REAL = [d for d in ALL if d.kind != "c"]


@pytest.mark.parametrize("name", ["add", "multiply"])
def test_binary_promotion_matches_numpy(name):
    f = getattr(ef, name)
    for d1 in ALL:
        for d2 in ALL:
            b1, b2, res = tu._find_buf_dtype2(d1, d2, f.result_type_resolver_fn_, f.acceptance_fn_)
            exp = np.promote_types(d1, d2)
            assert res == exp, (d1, d2, res, exp)
            assert (b1 or d1) == exp and (b2 or d2) == exp


def test_divide_promotion():
    f = ef.divide
    for d1 in REAL:
        for d2 in REAL:
            _, _, res = tu._find_buf_dtype2(d1, d2, f.result_type_resolver_fn_, f.acceptance_fn_)
            exp = np.true_divide(np.ones(1, d1), np.ones(1, d2)).dtype
            assert res == exp, (d1, d2, res, exp)


def test_comparison_promotion_and_mixed_sign_ints():
    f = ef.less
    i8, u8 = np.dtype("i8"), np.dtype("u8")
    assert tu._find_buf_dtype2(i8, u8, f.result_type_resolver_fn_, f.acceptance_fn_) == (None, None, np.dtype("?"))
    for d1 in REAL:
        for d2 in REAL:
            _, _, res = tu._find_buf_dtype2(d1, d2, f.result_type_resolver_fn_, f.acceptance_fn_)
            assert res == np.dtype("?")


def test_unary_promotion():
    for name in ("exp", "log", "sqrt"):
        f = getattr(ef, name)
        for d in REAL:
            buf, res = tu._find_buf_dtype(d, f.result_type_resolver_fn_, f.acceptance_fn_)
            exp = getattr(np, name)(np.ones(1, d)).dtype
            assert res == exp, (name, d, res, exp)
    with pytest.raises(ValueError, match="not supported for inputs of data type bool"):
        tu._find_buf_dtype(np.dtype("?"), ef.negative.result_type_resolver_fn_, ef.negative.acceptance_fn_)
    # erf keeps f4/f8 and widens f2 to f4
    assert tu._find_buf_dtype(np.dtype("f2"), ef.erf.result_type_resolver_fn_) == (None, np.dtype("f4"))
    assert tu._find_buf_dtype(np.dtype("i4"), ef.erf.result_type_resolver_fn_)[1] == np.dtype("f8")


def test_weak_python_scalars_follow_nep50():
    f4, i4, u1 = np.dtype("f4"), np.dtype("i4"), np.dtype("u1")
    assert tu._resolve_weak_types(f4, tu.WeakFloatingType(2.5)) == (f4, f4)
    assert tu._resolve_weak_types(i4, tu.WeakFloatingType(2.5)) == (i4, np.dtype("f8"))
    assert tu._resolve_weak_types(tu.WeakIntegralType(3), f4) == (f4, f4)
    assert tu._resolve_weak_types(np.dtype("?"), tu.WeakIntegralType(3)) == (np.dtype("?"), np.dtype("i8"))
    assert tu._resolve_weak_types(f4, tu.WeakComplexType(1j)) == (f4, np.dtype("c8"))
    assert tu._resolve_weak_types(np.dtype("f8"), tu.WeakComplexType(1j)) == (np.dtype("f8"), np.dtype("c16"))
    # comparisons/divide: an out-of-range Python int keeps its own minimal type
    assert tu._resolve_weak_types_all_py_ints(u1, tu.WeakIntegralType(-1)) == (u1, np.dtype("i1"))
    assert tu._resolve_weak_types_all_py_ints(u1, tu.WeakIntegralType(7)) == (u1, u1)
    with pytest.raises(ValueError):
        tu._resolve_weak_types(tu.WeakIntegralType(1), tu.WeakIntegralType(2))


def test_in_place_promotion():
    q = ef.add.result_type_resolver_fn_
    assert tu._find_buf_dtype_in_place_op(np.dtype("f4"), np.dtype("f4"), q) == (None, np.dtype("f4"))
    assert tu._find_buf_dtype_in_place_op(np.dtype("f4"), np.dtype("i4"), q) == (np.dtype("f4"), np.dtype("f4"))
    assert tu._find_buf_dtype_in_place_op(np.dtype("i4"), np.dtype("f4"), q) == (None, None)


def test_default_accumulation_types():
    exp = {"?": "i8", "i1": "i8", "i4": "i8", "i8": "i8", "u1": "u8", "u8": "u8", "f2": "f2", "f4": "f4",
           "f8": "f8", "c8": "c8"}
    for k, v in exp.items():
        assert tu._default_accumulation_dtype(np.dtype(k)) == np.dtype(v)
        assert np.sum(np.ones(2, k)).dtype == np.dtype(v) or k == "f2"


def test_broadcast_shapes():
    assert _broadcast_shape_impl([(64, 1024, 4096), (64, 1, 4096)]) == (64, 1024, 4096)
    assert _broadcast_shape_impl([(6, 1), (6,)]) == (6, 6)
    assert _broadcast_shape_impl([(), (3, 0)]) == (3, 0)
    with pytest.raises(ValueError, match="could not be broadcast"):
        _broadcast_shape_impl([(10, 10), (3,)])


def test_basic_slicing_matches_numpy():
    rng = np.random.default_rng(0)
    a = np.arange(4 * 5 * 6).reshape(4, 5, 6)
    es = tuple(s // a.itemsize for s in a.strides)
    keys = [np.s_[1], np.s_[:, 2], np.s_[::-1], np.s_[1:3, ::2, ::-2], np.s_[..., 1], np.s_[None, 1, ..., None],
            np.s_[3:1], np.s_[-1, -2, -3], np.s_[:, :, 10:], np.s_[::-3, 4:0:-2]]
    for key in keys:
        shape, strides, off, adv = basic_slice_meta(key, a.shape, es)
        v = a[key]
        assert not adv and shape == v.shape
        if v.size:
            got = np.lib.stride_tricks.as_strided(a.ravel()[off:], shape, tuple(s * a.itemsize for s in strides))
            np.testing.assert_array_equal(got, v)
    with pytest.raises(IndexError):
        basic_slice_meta(np.s_[4], a.shape, es)
    with pytest.raises(IndexError):
        basic_slice_meta(np.s_[0, 0, 0, 0], a.shape, es)
    assert basic_slice_meta(np.array([0, 1]), a.shape, es)[3] is True


def test_contiguity_flags_match_numpy():
    a = np.zeros((3, 4, 5))
    views = [a, a.T, a[:, ::2], a[::-1], a[:, :1, :], a[1:2], np.zeros((3, 1, 5)).transpose(1, 0, 2),
             np.zeros((0, 4)), np.zeros(()), np.zeros(7)[::2], np.zeros((1, 1, 6))]
    for v in views:
        es = tuple(s // v.itemsize for s in v.strides)
        fl = _contig_flags(v.shape, es)
        assert bool(fl & 1) == v.flags.c_contiguous and bool(fl & 2) == v.flags.f_contiguous, (v.shape, es)


def test_reshape_without_copy_rule():
    assert _reshape_strides((3, 4), (4, 1), (12,)) == (1,)
    assert _reshape_strides((3, 4), (1, 3), (12,)) is None          # transposed: needs a copy
    assert _reshape_strides((6, 4), (8, 1), (2, 3, 4)) == (24, 8, 1)  # row-strided, rows split
    assert _reshape_strides((6, 4), (8, 1), (24,)) is None
