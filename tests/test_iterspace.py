"""Iteration-space algebra of the C ABI, pinned against the reference's own
simplifier (oracle/_ref, compiled from its SYCL-free header) and against a
brute-force enumeration of the visited displacements."""

import ctypes as C

import numpy as np
import pytest

from dpnp_b200 import _lib
from dpnp_b200.tensor import _tensor_impl as ti
from oracle import dpnp_oracle as orc


def random_space(rng, narrays, nd):
    """Shapes/strides of views one could build from dense arrays: permutations,
    steps, reversals and broadcast (stride 0) dimensions."""
    shape = [int(v) for v in rng.integers(1, 5, size=nd)]
    strides = []
    for _ in range(narrays):
        perm = rng.permutation(nd)
        dense = [0] * nd
        acc = 1
        for d in perm[::-1]:
            dense[d] = acc
            acc *= shape[d] * int(rng.integers(1, 3))
        st = []
        for d in range(nd):
            r = rng.random()
            if r < 0.15:
                st.append(0)
            elif r < 0.35:
                st.append(-dense[d])
            else:
                st.append(dense[d])
        strides.append(st)
    return shape, strides


@pytest.mark.parametrize("narrays", [1, 2, 3, 4])
def test_simplify_visits_the_same_displacements(narrays):
    rng = np.random.default_rng(narrays)
    for _ in range(300):
        nd = int(rng.integers(1, 6))
        shape, strides = random_space(rng, narrays, nd)
        sh, sts, offs = ti._contract_iter_n(shape, *strides)
        assert len(sh) <= nd
        before = orc.displacement_set(shape, strides)
        after = orc.displacement_set(sh, sts, offs)
        assert before == after, (shape, strides, sh, sts, offs)


@pytest.mark.parametrize("narrays", [1, 2, 3, 4])
def test_simplify_equals_the_reference_implementation(narrays):
    if orc.ref_strided_iters() is None:
        pytest.skip("oracle/_ref was not built (reference tree absent)")
    rng = np.random.default_rng(100 + narrays)
    for _ in range(500):
        nd = int(rng.integers(2, 7))  # the reference's functions return at once below 2 dimensions
        shape, strides = random_space(rng, narrays, nd)
        got = ti._contract_iter_n(shape, *strides)
        ref = orc.simplify_ref(shape, strides)
        assert got[0] == ref[0] and got[1] == ref[1] and got[2] == ref[2], (shape, strides, got, ref)


def test_simplify_examples():
    # dense C array collapses to one dimension
    assert ti._contract_iter([3, 4, 5], [20, 5, 1]) == ([60], [1], 0)
    # fully reversed array: one dimension, offset at the last element
    assert ti._contract_iter([3, 4], [-4, -1]) == ([12], [1], -11)
    # transposed operand next to a dense result cannot collapse
    sh, sts, offs = ti._contract_iter_n([64, 8, 16], [1, 1024, 64], [16, 0, 1], [128, 16, 1])
    assert sh == [64, 8, 16] and sts[2] == [128, 16, 1]
    # a broadcast scalar does not prevent collapsing
    sh, sts, offs = ti._contract_iter_n([7, 9], [9, 1], [0, 0], [9, 1])
    assert sh == [63] and sts == [[1], [0], [1]]


def test_compact_iteration_keeps_order():
    sh = (C.c_int64 * 3)(2, 3, 4)
    st = (C.c_int64 * 3)(12, 4, 1)
    n = C.c_int()
    _lib.check(_lib.lib.dpb_compact_iteration(3, sh, st, C.byref(n)))
    assert n.value == 1 and sh[0] == 24 and st[0] == 1
    sh = (C.c_int64 * 3)(2, 3, 4)
    st = (C.c_int64 * 3)(1, 2, 6)  # F order: nothing merges in C order
    _lib.check(_lib.lib.dpb_compact_iteration(3, sh, st, C.byref(n)))
    assert n.value == 3
    if orc.ref_strided_iters() is not None:
        rng = np.random.default_rng(5)
        for _ in range(300):
            nd = int(rng.integers(2, 6))
            shape, strides = random_space(rng, 1, nd)
            a = (C.c_int64 * nd)(*shape), (C.c_int64 * nd)(*strides[0])
            b = (C.c_int64 * nd)(*shape), (C.c_int64 * nd)(*strides[0])
            _lib.check(_lib.lib.dpb_compact_iteration(nd, a[0], a[1], C.byref(n)))
            m = orc.ref_strided_iters().ref_compact(nd, b[0], b[1])
            assert n.value == m and list(a[0][:m]) == list(b[0][:m]) and list(a[1][:m]) == list(b[1][:m])


def _desc(ptr, shape, strides, dtype="f4"):
    nd = len(shape)
    sh = (C.c_int64 * max(nd, 1))(*shape)
    st = (C.c_int64 * max(nd, 1))(*strides)
    d = _lib.dpb_array()
    d.data, d.nd, d.typenum, d.flags, d.device = ptr, nd, _lib.typenum_of(dtype), 7, 0
    d.shape = C.cast(sh, C.POINTER(C.c_int64))
    d.strides = C.cast(st, C.POINTER(C.c_int64))
    return d, (sh, st)


def test_overlap_and_same_logical_tensor():
    out = C.c_int()
    a, ka = _desc(4096, (10, 10), (10, 1))
    b, kb = _desc(4096 + 4 * 50, (5, 10), (10, 1))      # second half of a
    c, kc = _desc(4096 + 4 * 100, (10, 10), (10, 1))    # right after a
    d, kd = _desc(4096, (10, 10), (10, 1))
    e, ke = _desc(4096 + 4 * 99, (10, 10), (-10, -1))   # a reversed: same bytes
    for x, y, exp in ((a, b, 1), (a, c, 0), (a, d, 1), (a, e, 1)):
        _lib.check(_lib.lib.dpb_array_overlap(C.byref(x), C.byref(y), C.byref(out)))
        assert out.value == exp
    for x, y, exp in ((a, d, 1), (a, b, 0), (a, e, 0)):
        _lib.check(_lib.lib.dpb_same_logical_tensors(C.byref(x), C.byref(y), C.byref(out)))
        assert out.value == exp
    z, kz = _desc(4096, (0, 10), (10, 1))
    _lib.check(_lib.lib.dpb_array_overlap(C.byref(a), C.byref(z), C.byref(out)))
    assert out.value == 0
