"""`lt.cuda`: device queries, the TF32 switch, allocator statistics, CUDA-graph capture.

Mirrors src/bindings/python_bindings.cpp:175-199 (`is_available, set_tf32_enabled, is_tf32_enabled,
memory_allocated`) and the stream-capture graph entry points of the reference backend
(src/backend/gpu_native/entrypoint.cu:162-215).  `use_caching_allocator()` routes every PyTorch CUDA
allocation through the native stream-aware caching allocator of liblt_cuda.so.
"""
from __future__ import annotations

import contextlib
import ctypes
import os

import torch

_tf32 = [True]


def is_available() -> bool:
    return torch.cuda.is_available()


def set_tf32_enabled(flag: bool) -> None:
    _tf32[0] = bool(flag)
    torch.backends.cuda.matmul.allow_tf32 = bool(flag)
    torch.backends.cudnn.allow_tf32 = bool(flag)


def is_tf32_enabled() -> bool:
    return _tf32[0]


def memory_allocated() -> int:
    return torch.cuda.memory_allocated() if torch.cuda.is_available() else 0


def device_count() -> int:
    return torch.cuda.device_count()


_installed = [False]


def use_caching_allocator() -> bool:
    """Install the native allocator as PyTorch's CUDA allocator. Must run before the first CUDA allocation.

    Blocks are cached per (device, stream) and reused in stream order.  A temporary that another stream also uses
    must be announced with `lt.cuda.record_stream(tensor, stream)`: PyTorch does not forward
    `tensor.record_stream` to a pluggable allocator from Python.  While a stream records a CUDA graph the allocator
    serves requests from its cache only (it never calls cudaMalloc inside a capture); run the region once eagerly
    first."""
    if _installed[0]:
        return True
    from ._native import _LIB
    path = os.path.join(_LIB, "liblt_cuda.so")
    alloc = torch.cuda.memory.CUDAPluggableAllocator(path, "lt_cuda_alloc", "lt_cuda_free")
    torch.cuda.memory.change_current_allocator(alloc)
    _installed[0] = True
    return True


def record_stream(t: torch.Tensor, stream: "torch.cuda.Stream") -> None:
    """`t` is used on `stream` (not the stream it was allocated on): keep its memory from being handed out again,
    after `t` is freed, until the work queued on `stream` so far has finished.  Works with PyTorch's own allocator
    (tensor.record_stream) and with the native one (lt_cuda_record_stream)."""
    t.record_stream(stream)
    if _installed[0]:
        from ._native import cuda_lib
        cuda_lib().lt_cuda_record_stream(ctypes.c_void_p(t.untyped_storage().data_ptr()), ctypes.c_void_p(stream.cuda_stream))


def allocator_stats() -> dict:
    from ._native import cuda_lib
    out = (ctypes.c_uint64 * 5)()
    cuda_lib().lt_cuda_alloc_stats(out)
    return dict(zip(("cached_bytes", "allocated_bytes", "peak_bytes", "hits", "misses"), [int(v) for v in out]))


def empty_cache() -> None:
    if torch.cuda.is_available():
        torch.cuda.empty_cache()
        if _installed[0]:
            from ._native import cuda_lib
            cuda_lib().lt_cuda_empty_cache()


class CapturedGraph:
    """Capture the kernels launched inside `with g.capture():` on a side stream into a CUDA graph; `replay()`
    launches the whole graph.  Native kernels are captured like any other launch because they run on the
    current torch stream."""

    def __init__(self):
        self._g = torch.cuda.CUDAGraph()

    @contextlib.contextmanager
    def capture(self):
        with torch.cuda.graph(self._g):
            yield self

    def replay(self):
        self._g.replay()


class NativeGraph:
    """The same through the native runtime (cudaStreamBeginCapture / Instantiate / Launch on a given stream);
    used when no torch allocation happens inside the captured region."""

    def __init__(self):
        from ._native import cuda_lib
        self._lib = cuda_lib()
        self._lib.lt_graph_end_capture.restype = ctypes.c_void_p
        self._exec = None

    def begin(self, stream: torch.cuda.Stream):
        rc = self._lib.lt_graph_begin_capture(ctypes.c_void_p(stream.cuda_stream))
        if rc != 0:
            raise RuntimeError("cudaStreamBeginCapture failed: %d" % rc)

    def end(self, stream: torch.cuda.Stream):
        err = ctypes.c_int(0)
        self._exec = self._lib.lt_graph_end_capture(ctypes.c_void_p(stream.cuda_stream), ctypes.byref(err))
        if not self._exec:
            raise RuntimeError("graph capture failed: %d" % err.value)

    def launch(self, stream: torch.cuda.Stream):
        rc = self._lib.lt_graph_launch(ctypes.c_void_p(self._exec), ctypes.c_void_p(stream.cuda_stream))
        if rc != 0:
            raise RuntimeError("cudaGraphLaunch failed: %d" % rc)

    def __del__(self):
        try:
            if self._exec:
                self._lib.lt_graph_destroy(ctypes.c_void_p(self._exec))
        except Exception:
            pass
