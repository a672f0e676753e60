"""The double-precision erf of the kernels (dpnp_b200/csrc/ew_erf.cuh) compiled for the HOST and
measured against correctly rounded values (mpmath).  The function is the same source on the host and
on the device (the series below 1/16, the table-driven Taylor step up to 6); only the table's memory
space and the way the index is read from the rounded sum differ.  tests/test_gpu_elementwise.py repeats
the measurement on the device.  With an error below 1 ulp, any reference whose erf is accurate to 1 ulp
is at most 2 ulp away."""

import ctypes as C
import os
import shutil
import subprocess

import numpy as np
import pytest

from oracle import dpnp_oracle as orc

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "host_harness", "erf_host.cu")


@pytest.fixture(scope="module")
def erf_host(tmp_path_factory):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("nvcc is needed to build the host harness")
    out = str(tmp_path_factory.mktemp("erf") / "liberf_host.so")
    cmd = [nvcc, "-O1", "-std=c++17", "-fmad=false", "--expt-relaxed-constexpr", "-shared", "-Xcompiler", "-fPIC",
           "-Wno-deprecated-gpu-targets", "-x", "cu", SRC, "-o", out]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    assert proc.returncode == 0, proc.stderr
    lib = C.CDLL(out)

    def run(x):
        x = np.ascontiguousarray(x, dtype="f8")
        res = np.empty_like(x)
        lib.erf_f64_host(C.c_long(x.size), x.ctypes.data_as(C.c_void_p), res.ctypes.data_as(C.c_void_p))
        return res
    return run


def test_erf_is_within_one_ulp_of_the_correctly_rounded_value(erf_host):
    rng = np.random.default_rng(0)
    edges = np.arange(0.5, 6.0, 0.125)
    p, k, t = rng.uniform(10, 50, 2000), rng.uniform(10, 50, 2000), rng.uniform(1, 2, 2000)
    a, b, z = np.log(p / k), t * -0.1, t * 0.08           # the chain's arguments of erf: w1, w2
    w1, w2 = (a - b + 0.25 * z) / np.sqrt(z), (a - b - 0.25 * z) / np.sqrt(z)
    x = np.concatenate([rng.uniform(-6, 6, 6000), rng.uniform(-0.5, 0.5, 6000), rng.uniform(0.4, 0.7, 1000),
                        edges, np.nextafter(edges, 0), np.nextafter(edges, 10), -edges, w1, w2,
                        [1e-300, 1e-20, 5.9, 5.99, 0.5, -0.5, 4.5]])
    ulp = orc.ulp_distance(erf_host(x), orc.mp_reference("erf", x))
    assert ulp.max() < 1.0, (ulp.max(), x[ulp.argmax()])
    assert ulp.mean() < 0.35


def test_erf_special_values(erf_host):
    got = erf_host(np.array([np.nan, np.inf, -np.inf, 0.0, -0.0, 6.0, -6.0, 30.0, 5e-324]))
    assert np.isnan(got[0]) and got[1] == 1.0 and got[2] == -1.0
    assert got[3] == 0.0 and not np.signbit(got[3]) and got[4] == 0.0 and np.signbit(got[4])
    assert got[5] == 1.0 and got[6] == -1.0 and got[7] == 1.0
    assert got[8] == 5e-324 * 1.0 or got[8] == 1e-323      # 2/sqrt(pi) times the smallest subnormal
    # odd function, monotone across the table intervals and the switch between the two forms
    x = np.linspace(0.0, 6.0, 48001)
    y = erf_host(x)
    assert (np.diff(y) >= 0).all() and np.array_equal(erf_host(-x), -y)
