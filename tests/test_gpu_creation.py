"""Device-side creation (arange, linspace) and DLPack exchange."""

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_arange_is_written_on_the_device():
    import dpnp_b200 as dp
    from dpnp_b200 import _lib

    for args, kw in (((10,), {}), ((2, 30, 3), {}), ((5, -20, -4), {}), ((0.5, 9.25, 0.75), {}),
                     ((10,), {"dtype": "f4"}), ((0, 300, 7), {"dtype": "u1"}), ((3, 3), {}), ((5, 2), {}),
                     ((0, 1 << 20), {"dtype": "i4"}), ((0.0, 1.0, 1e-5), {}), ((-3, 40), {"dtype": "i8"})):
        got = dp.arange(*args, **kw)
        ref = np.arange(*args, **kw)
        assert got.shape == ref.shape and got.dtype == ref.dtype, (args, kw)
        if ref.size:
            assert _lib.last_kernel() == "sequence_step"
        if ref.dtype.kind == "f":
            np.testing.assert_allclose(got.asnumpy(), ref, rtol=1e-6 if ref.dtype == np.float32 else 1e-14)
        else:
            np.testing.assert_array_equal(got.asnumpy(), ref)
    with pytest.raises(ValueError):
        dp.arange(5, dtype="?")
    np.testing.assert_array_equal(dp.arange(2, dtype="?").asnumpy(), [False, True])


def test_linspace_matches_the_affine_formula():
    import dpnp_b200 as dp

    for start, stop, num, kw in ((0, 1, 11, {}), (-3.5, 12.25, 1000, {}), (5, -5, 7, {"endpoint": False}),
                                 (0, 10, 1, {}), (1, 2, 0, {}), (0, 1, 50, {"dtype": "f4"}),
                                 (0, 100, 11, {"dtype": "i4"})):
        got = dp.linspace(start, stop, num, **kw)
        ref = np.linspace(start, stop, num, **kw)
        assert got.shape == ref.shape and got.dtype == ref.dtype
        # element i is start*(den-i)/den + stop*i/den with two fused multiply-adds
        den = max((num - 1) if kw.get("endpoint", True) else num, 1)
        if ref.dtype.kind == "f":
            i = np.arange(num, dtype="f8")
            w, wc = ((den - i) / den).astype(ref.dtype), (i / den).astype(ref.dtype)
            exact = ref.dtype.type(start) * w.astype(np.longdouble) + ref.dtype.type(stop) * wc.astype(np.longdouble)
            eps = np.finfo(ref.dtype).eps
            assert np.all(np.abs(got.asnumpy() - exact) <= 2 * eps * (abs(start) + abs(stop)) + 1e-300)
            if num > 1 and kw.get("endpoint", True):
                assert got.asnumpy()[0] == start and got.asnumpy()[-1] == stop
        else:
            np.testing.assert_array_equal(got.asnumpy(), ref)
    with pytest.raises(ValueError):
        dp.linspace(0, 1, -1)
    with pytest.raises(TypeError):
        dp.linspace(0, 1, 5, endpoint="yes")


def test_dlpack_round_trip_with_torch_shares_memory():
    import torch

    import dpnp_b200 as dp

    x = dp.asarray(np.arange(24, dtype="f4").reshape(4, 6))
    assert x.__dlpack_device__() == (2, 0)
    t = torch.from_dlpack(x)                                  # export: no copy
    assert t.is_cuda and t.shape == (4, 6) and t.data_ptr() == x.get_array()._ptr
    t.mul_(2)
    torch.cuda.synchronize()
    np.testing.assert_array_equal(x.asnumpy(), np.arange(24, dtype="f4").reshape(4, 6) * 2)
    tv = torch.from_dlpack(x[1:, ::2])                        # strided views keep their strides
    assert tuple(tv.stride()) == (6, 2) and tv.shape == (3, 3)
    np.testing.assert_array_equal(tv.cpu().numpy(), x.asnumpy()[1:, ::2])

    src = torch.arange(30, dtype=torch.int64, device="cuda").reshape(5, 6)
    torch.cuda.synchronize()
    y = dp.from_dlpack(src)                                   # import: no copy
    assert y.dtype == np.dtype("i8") and y.shape == (5, 6) and y.get_array()._ptr == src.data_ptr()
    np.testing.assert_array_equal((y + 1).asnumpy(), np.arange(30).reshape(5, 6) + 1)
    np.testing.assert_array_equal(dp.sum(y, axis=0).asnumpy(), np.arange(30).reshape(5, 6).sum(axis=0))
    yt = dp.from_dlpack(src.t())
    assert yt.shape == (6, 5) and not yt.flags.c_contiguous
    np.testing.assert_array_equal(yt.asnumpy(), np.arange(30).reshape(5, 6).T)
    del src                                                   # the import keeps the memory alive
    np.testing.assert_array_equal(y.asnumpy(), np.arange(30).reshape(5, 6))
    z = dp.from_dlpack(dp.asarray(np.ones(3)))                # own arrays through the protocol
    np.testing.assert_array_equal(z.asnumpy(), np.ones(3))
    with pytest.raises(BufferError):
        dp.from_dlpack(torch.ones(3))                         # host memory is refused
    c = dp.from_dlpack(torch.ones(4, device="cuda"), copy=True)
    assert c.asnumpy().sum() == 4
