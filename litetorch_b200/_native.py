"""Build and load the native libraries.

Two shared objects live in ``litetorch_b200/_lib``:

* ``liblt_cuda.so``  - every sm_100a kernel plus the CUDA-side runtime (allocator, graph capture,
  NVRTC JIT). Built with ``nvcc -gencode arch=compute_100a,code=sm_100a``.
* ``liblt_host.so``  - the host runtime in C++17 with no CUDA dependency: checkpoint formats,
  data loader, serving scheduler, rendezvous store, JIT expression trees, thread pool.

Both export plain C symbols and are called through ``ctypes``; nothing is JIT-compiled at import
time.  The reference ships one pybind11 module plus a dlopen'ed GPU library
(src/backend/backend.cpp:61-341); here the split is host/CUDA so that CPU-only processes (gloo
ranks, the data-loader workers, tests without a GPU) never touch the CUDA runtime.
"""
from __future__ import annotations

import ctypes
import glob
import os
import shutil
import subprocess
import sys
import threading
from concurrent.futures import ThreadPoolExecutor

_PKG = os.path.dirname(os.path.abspath(__file__))
_ROOT = os.path.dirname(_PKG)
_CSRC = os.path.join(_ROOT, "csrc")
_LIB = os.path.join(_PKG, "_lib")
_OBJ = os.path.join(_ROOT, "build", "obj")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-Wall", "-pthread"]


def _nvcc() -> str:
    for c in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if c and os.path.exists(c):
            return c
    raise RuntimeError("nvcc not found")


def _newest(paths) -> float:
    return max((os.path.getmtime(p) for p in paths), default=0.0)


def _compile_one(cmd, out):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("compile failed: %s\n%s\n%s" % (" ".join(cmd), r.stdout, r.stderr))
    return out


def cuda_sources():
    return sorted(glob.glob(os.path.join(_CSRC, "kernels", "**", "*.cu"), recursive=True)) + sorted(
        glob.glob(os.path.join(_CSRC, "cuda_runtime", "*.cu")))


def host_sources():
    return sorted(glob.glob(os.path.join(_CSRC, "runtime", "*.cpp")))


def build_cuda(force: bool = False, verbose: bool = False) -> str:
    """Compile every .cu under csrc/ for sm_100a and link liblt_cuda.so (cross-compiles without a GPU)."""
    os.makedirs(_LIB, exist_ok=True)
    os.makedirs(_OBJ, exist_ok=True)
    out = os.path.join(_LIB, "liblt_cuda.so")
    srcs = cuda_sources()
    hdrs = glob.glob(os.path.join(_CSRC, "**", "*.cuh"), recursive=True) + glob.glob(
        os.path.join(_CSRC, "**", "*.h"), recursive=True)
    hdr_time = _newest(hdrs)
    nvcc = _nvcc()
    jobs, objs = [], []
    for s in srcs:
        o = os.path.join(_OBJ, os.path.relpath(s, _CSRC).replace(os.sep, "_") + ".o")
        objs.append(o)
        if force or not os.path.exists(o) or os.path.getmtime(o) < max(os.path.getmtime(s), hdr_time):
            cmd = [nvcc] + NVCC_FLAGS + ["-I", os.path.join(_CSRC, "kernels"), "-I", _CSRC, "-c", s, "-o", o]
            jobs.append((cmd, o))
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for o in ex.map(lambda j: _compile_one(*j), jobs):
                if verbose:
                    print("compiled", o)
    if jobs or not os.path.exists(out) or os.path.getmtime(out) < _newest(objs):
        cmd = [nvcc, "-shared", "-o", out + ".tmp"] + objs + ["-ldl"]
        _compile_one(cmd, out)
        os.replace(out + ".tmp", out)      # a reader never sees a half-written library
    return out


def build_host(force: bool = False, verbose: bool = False) -> str:
    """Compile the CUDA-free host runtime into liblt_host.so."""
    os.makedirs(_LIB, exist_ok=True)
    os.makedirs(_OBJ, exist_ok=True)
    out = os.path.join(_LIB, "liblt_host.so")
    srcs = host_sources()
    hdrs = glob.glob(os.path.join(_CSRC, "runtime", "*.h"))
    hdr_time = _newest(hdrs)
    cxx = shutil.which("g++") or "g++"
    jobs, objs = [], []
    for s in srcs:
        o = os.path.join(_OBJ, "host_" + os.path.basename(s) + ".o")
        objs.append(o)
        if force or not os.path.exists(o) or os.path.getmtime(o) < max(os.path.getmtime(s), hdr_time):
            jobs.append(([cxx] + CXX_FLAGS + ["-I", os.path.join(_CSRC, "runtime"), "-c", s, "-o", o], o))
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for o in ex.map(lambda j: _compile_one(*j), jobs):
                if verbose:
                    print("compiled", o)
    if srcs and (jobs or not os.path.exists(out) or os.path.getmtime(out) < _newest(objs)):
        _compile_one([cxx, "-shared", "-pthread", "-o", out + ".tmp"] + objs + ["-lrt", "-ldl"], out)
        os.replace(out + ".tmp", out)
    return out


def build_all(force: bool = False, verbose: bool = False):
    return build_host(force, verbose), build_cuda(force, verbose)


_lock = threading.Lock()
_cuda = None
_host = None


class NativeLibraryMissing(RuntimeError):
    pass


def cuda_lib() -> ctypes.CDLL:
    """liblt_cuda.so; raises loudly when it has not been built (no silent fallback on a GPU box)."""
    global _cuda
    if _cuda is not None:
        return _cuda
    with _lock:
        if _cuda is None:
            path = os.path.join(_LIB, "liblt_cuda.so")
            if not os.path.exists(path):
                raise NativeLibraryMissing(
                    "liblt_cuda.so is not built; run `python -c 'import __graft_entry__ as g; g.build()'` "
                    "or `python -m litetorch_b200._native`")
            _cuda = ctypes.CDLL(path, mode=ctypes.RTLD_GLOBAL)
    return _cuda


def host_lib() -> ctypes.CDLL:
    """liblt_host.so; built on first use if absent (g++ only, a few seconds)."""
    global _host
    if _host is not None:
        return _host
    with _lock:
        if _host is None:
            path = os.path.join(_LIB, "liblt_host.so")
            if not os.path.exists(path):
                build_host()
            _host = ctypes.CDLL(path, mode=ctypes.RTLD_GLOBAL)
    return _host


def have_cuda_lib() -> bool:
    return os.path.exists(os.path.join(_LIB, "liblt_cuda.so"))


if __name__ == "__main__":
    print(build_all(force="--force" in sys.argv, verbose=True))
