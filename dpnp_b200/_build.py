"""In-tree build of libdpnp_b200.so with nvcc for sm_100a.

``python dpnp_b200/_build.py`` compiles every source under ``csrc/`` into an
object file (in parallel, skipping objects newer than all sources and headers)
and links them into ``dpnp_b200/libdpnp_b200.so``.  The CUDA runtime is linked
statically, so the library needs only the driver at run time.
"""

from __future__ import annotations

import os
import re
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ_DIR = os.path.join(HERE, "build")
LIB_PATH = os.path.join(HERE, "libdpnp_b200.so")

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "-fmad=false",  # every multiply and add rounds on its own, as the per-op reference kernels do
    "--expt-relaxed-constexpr",
    "-Xcompiler",
    "-fPIC",
    "-diag-suppress=128",  # "loop is not reachable": if-constexpr branches that return early
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC or add it to PATH")


def _sources() -> list[str]:
    return sorted(
        os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cu", ".cpp"))
    )


_INCLUDE_RE = re.compile(r'^\s*#\s*include\s+"([^"]+)"', re.M)


def _deps_mtime(path: str, seen: dict[str, float] | None = None) -> float:
    """Newest modification time of `path` and of every header it includes."""
    seen = {} if seen is None else seen
    path = os.path.normpath(path)
    if path in seen:
        return seen[path]
    seen[path] = newest = os.path.getmtime(path)
    with open(path, "r", encoding="utf-8") as fh:
        text = fh.read()
    for inc in _INCLUDE_RE.findall(text):
        cand = os.path.normpath(os.path.join(os.path.dirname(path), inc))
        if os.path.exists(cand):
            newest = max(newest, _deps_mtime(cand, seen))
    seen[path] = newest
    return newest


def _compile_one(nvcc: str, src: str, obj: str, extra: list[str]) -> tuple[str, int, str]:
    cmd = [nvcc, *NVCC_FLAGS, *extra, "-x", "cu", "-c", src, "-o", obj]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    return src, proc.returncode, proc.stdout + proc.stderr


def build(force: bool = False, verbose: bool = False, jobs: int | None = None,
          ptxas_info: bool = False) -> str:
    """Compile and link the library; returns its path."""
    nvcc = _nvcc()
    os.makedirs(OBJ_DIR, exist_ok=True)
    extra = ["-Xptxas", "-v"] if ptxas_info else []
    todo = []
    objs = []
    for src in _sources():
        obj = os.path.join(OBJ_DIR, os.path.basename(src) + ".o")
        objs.append(obj)
        if (
            force
            or ptxas_info
            or not os.path.exists(obj)
            or os.path.getmtime(obj) < _deps_mtime(src)
        ):
            todo.append((src, obj))
    if todo:
        jobs = jobs or max(1, (os.cpu_count() or 2))
        with ThreadPoolExecutor(max_workers=jobs) as pool:
            results = list(pool.map(lambda so: _compile_one(nvcc, so[0], so[1], extra), todo))
        failed = False
        for src, rc, out in results:
            if verbose or rc != 0 or ptxas_info:
                sys.stderr.write(f"[nvcc] {os.path.basename(src)} -> rc={rc}\n{out}\n")
            failed = failed or rc != 0
        if failed:
            raise RuntimeError("compilation of libdpnp_b200 failed")
    if todo or not os.path.exists(LIB_PATH):
        link = [nvcc, "-shared", "-o", LIB_PATH, *objs, "-gencode",
                "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC"]
        proc = subprocess.run(link, capture_output=True, text=True)
        if proc.returncode != 0:
            sys.stderr.write(proc.stdout + proc.stderr)
            raise RuntimeError("link of libdpnp_b200.so failed")
    return LIB_PATH


def shim_path() -> str:
    import sysconfig

    return os.path.join(HERE, "_tensor_native" + (sysconfig.get_config_var("EXT_SUFFIX") or ".so"))


def build_shim(force: bool = False) -> str:
    """Compile the pybind11 shim (csrc/pyshim/tensor_native.cpp) with the host compiler and link
    it against libdpnp_b200.so, found at run time next to the module ($ORIGIN)."""
    import sysconfig

    import pybind11

    src = os.path.join(CSRC, "pyshim", "tensor_native.cpp")
    out = shim_path()
    header = os.path.join(os.path.dirname(HERE), "include", "dpnp_b200.h")
    if (not force and os.path.exists(out)
            and os.path.getmtime(out) >= max(os.path.getmtime(src), os.path.getmtime(header),
                                             os.path.getmtime(LIB_PATH))):
        return out
    cxx = os.environ.get("CXX") or shutil.which("g++") or "g++"
    cmd = [cxx, "-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden",
           "-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"],
           src, "-o", out, "-L", HERE, "-l:libdpnp_b200.so", "-Wl,-rpath,$ORIGIN"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        sys.stderr.write(proc.stdout + proc.stderr)
        raise RuntimeError("building the pybind11 shim failed")
    return out


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv,
                 ptxas_info="--ptxas" in sys.argv)
    print(path)
    print(build_shim(force="--force" in sys.argv))
