"""CUDA path against the known-answer cases lifted from the reference's tests."""

import numpy as np
import pytest

from tests._golden import apply_view, axis_of, load_cases

pytestmark = pytest.mark.gpu
CASES = load_cases()


def device_eval(c):
    import dpnp_b200 as dp

    order = c["params"].get("order", "C")
    x = dp.asarray(np.asfortranarray(c["x"]) if order == "F" else c["x"])
    x = apply_view(x, c["view"], dp)
    op, ax = c["op"], axis_of(c["params"])
    if op == "sum":
        return dp.sum(x, axis=ax, dtype=c["params"].get("dtype"))
    if op in ("max", "min"):
        return getattr(dp, op)(x, axis=ax, keepdims=c["params"].get("keepdims", False))
    if op in ("argmax", "argmin", "mean"):
        return getattr(dp, op)(x, axis=ax)
    if op == "where":
        views = c["params"]["views"]
        return dp.where(apply_view(dp.asarray(c["cond"]), views.get("cond", []), dp),
                        apply_view(x, views.get("x", []), dp),
                        apply_view(dp.asarray(c["y"]), views.get("y", []), dp))
    if op == "add":
        return dp.add(x, dp.asarray(c["y"]))
    if op in ("exp", "erf"):
        return getattr(dp, op)(x)
    raise AssertionError(op)


@pytest.mark.parametrize("c", CASES, ids=[c["name"] for c in CASES])
def test_device_matches_known_answer(c):
    got = device_eval(c).asnumpy()
    exp = c["expected"]
    assert got.shape == exp.shape
    assert got.dtype == exp.dtype
    if c["exact"]:
        np.testing.assert_array_equal(got, exp)
        if exp.dtype.kind == "f":
            ok = ~np.isnan(exp)
            np.testing.assert_array_equal(np.signbit(got)[ok], np.signbit(exp)[ok])
    else:
        tol = 8 * np.finfo(exp.dtype).resolution
        np.testing.assert_allclose(got, exp, rtol=tol, atol=tol)
