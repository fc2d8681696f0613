"""`NativeNccl`: NCCL collectives through the repository's own runtime (csrc/cuda_runtime/nccl_bridge.cu), bootstrapped
through the native TCP store - no `torch.distributed` involved.

    store = TCPStore("127.0.0.1", port, is_server=(rank == 0))
    comm = NativeNccl(store, rank, world)          # rank 0 publishes the 128-byte id, the others fetch it
    comm.all_reduce(t); comm.all_gather(out, t); comm.reduce_scatter(out, t); comm.broadcast(t, 0); comm.send(t, 1)

Operations are enqueued on the current torch CUDA stream and return at once (stream-ordered like any kernel launch).
The reference's counterpart is NCCLBridge (src/distributed/distributed.cpp:785-905).
"""
from __future__ import annotations

import ctypes
import os
import time
from ctypes import c_int, c_ulonglong, c_void_p

import torch

from .._native import cuda_lib

_DT = {torch.float32: 7, torch.float16: 6, torch.bfloat16: 9, torch.int32: 2, torch.int64: 4, torch.uint8: 1, torch.int8: 0,
       torch.float64: 8}
_OP = {"sum": 0, "prod": 1, "max": 2, "min": 3, "avg": 4}


def _lib():
    L = cuda_lib()
    if not getattr(L, "_lt_nccl_bound", False):
        L.lt_nccl_init.restype = c_void_p
        L.lt_nccl_init.argtypes = [c_void_p, c_int, c_int, ctypes.POINTER(c_int)]
        L.lt_nccl_unique_id.argtypes = [c_void_p]
        L.lt_nccl_destroy.argtypes = [c_void_p]
        L.lt_nccl_all_reduce.argtypes = [c_void_p, c_void_p, c_void_p, c_ulonglong, c_int, c_int, c_void_p]
        L.lt_nccl_all_gather.argtypes = [c_void_p, c_void_p, c_void_p, c_ulonglong, c_int, c_void_p]
        L.lt_nccl_reduce_scatter.argtypes = [c_void_p, c_void_p, c_void_p, c_ulonglong, c_int, c_int, c_void_p]
        L.lt_nccl_broadcast.argtypes = [c_void_p, c_void_p, c_void_p, c_ulonglong, c_int, c_int, c_void_p]
        L.lt_nccl_send.argtypes = [c_void_p, c_void_p, c_ulonglong, c_int, c_int, c_void_p]
        L.lt_nccl_recv.argtypes = [c_void_p, c_void_p, c_ulonglong, c_int, c_int, c_void_p]
        L._lt_nccl_bound = True
    return L


def nccl_version() -> int:
    """0 when libnccl cannot be opened, else its version code (2.28.9 -> 22809)."""
    return int(_lib().lt_nccl_version())


class NcclError(RuntimeError):
    pass


def _id_file():
    for k in ("LITETORCH_RENDEZVOUS_FILE", "NCCL_UNIQUE_ID_FILE"):
        v = os.environ.get(k, "")
        if v:
            return v + ".ncclid"
    return None


def publish_id_file(path: str, raw: bytes) -> None:
    """Rank 0 of the reference writes the 128-byte communicator id into the rendezvous file and the others poll for it
    (src/distributed/distributed.cpp:829-860).  Written to a temporary name and renamed, so that a reader never sees a
    partial id."""
    tmp = "%s.%d.tmp" % (path, os.getpid())
    with open(tmp, "wb") as f:
        f.write(raw)
        f.flush()
        os.fsync(f.fileno())
    os.replace(tmp, path)


def read_id_file(path: str, timeout_s: float = 120.0) -> bytes:
    t_end = time.monotonic() + timeout_s
    while True:
        try:
            with open(path, "rb") as f:
                raw = f.read()
            if len(raw) >= 128:
                return raw[:128]
        except OSError:
            pass
        if time.monotonic() > t_end:
            raise NcclError("no communicator id in %s after %.0f s" % (path, timeout_s))
        time.sleep(0.01)


class NativeNccl:
    def __init__(self, store, rank: int, world: int, key: str = "lt_nccl_id", timeout_s: float = 120.0):
        self._L = _lib()
        self.rank, self.world = rank, world
        if nccl_version() == 0:
            raise NcclError("libnccl.so.2 could not be opened")
        id_file = None if store is not None else _id_file()
        if store is None and id_file is None:
            raise NcclError("no store given and neither LITETORCH_RENDEZVOUS_FILE nor NCCL_UNIQUE_ID_FILE is set")
        if rank == 0:
            buf = (ctypes.c_char * 128)()
            rc = self._L.lt_nccl_unique_id(buf)
            if rc != 0:
                raise NcclError("ncclGetUniqueId failed: %d" % rc)
            raw = bytes(buf.raw)
            if store is not None:
                store.set(key, raw)
            else:
                publish_id_file(id_file, raw)
        elif store is not None:
            raw = store.get(key, timeout_s=timeout_s)
        else:
            raw = read_id_file(id_file, timeout_s)
        if len(raw) != 128:
            raise NcclError("rendezvous returned %d bytes for the communicator id" % len(raw))
        err = c_int(0)
        self._c = self._L.lt_nccl_init(raw, world, rank, ctypes.byref(err))
        if not self._c:
            raise NcclError("ncclCommInitRank failed: %d" % err.value)

    @staticmethod
    def _s():
        return c_void_p(torch.cuda.current_stream().cuda_stream)

    def _chk(self, rc, what):
        if rc != 0:
            raise NcclError("%s failed: ncclResult %d" % (what, rc))

    def all_reduce(self, t: torch.Tensor, op: str = "sum") -> torch.Tensor:
        assert t.is_cuda and t.is_contiguous()
        self._chk(self._L.lt_nccl_all_reduce(self._c, t.data_ptr(), t.data_ptr(), t.numel(), _DT[t.dtype], _OP[op], self._s()), "all_reduce")
        return t

    def all_gather(self, out: torch.Tensor, t: torch.Tensor) -> torch.Tensor:
        assert out.numel() == t.numel() * self.world and out.is_contiguous() and t.is_contiguous()
        self._chk(self._L.lt_nccl_all_gather(self._c, t.data_ptr(), out.data_ptr(), t.numel(), _DT[t.dtype], self._s()), "all_gather")
        return out

    def reduce_scatter(self, out: torch.Tensor, t: torch.Tensor, op: str = "sum") -> torch.Tensor:
        assert t.numel() == out.numel() * self.world and out.is_contiguous() and t.is_contiguous()
        self._chk(self._L.lt_nccl_reduce_scatter(self._c, t.data_ptr(), out.data_ptr(), out.numel(), _DT[t.dtype], _OP[op], self._s()),
                  "reduce_scatter")
        return out

    def broadcast(self, t: torch.Tensor, root: int) -> torch.Tensor:
        self._chk(self._L.lt_nccl_broadcast(self._c, t.data_ptr(), t.data_ptr(), t.numel(), _DT[t.dtype], root, self._s()), "broadcast")
        return t

    def send(self, t: torch.Tensor, peer: int) -> None:
        self._chk(self._L.lt_nccl_send(self._c, t.data_ptr(), t.numel(), _DT[t.dtype], peer, self._s()), "send")

    def recv(self, t: torch.Tensor, peer: int) -> torch.Tensor:
        self._chk(self._L.lt_nccl_recv(self._c, t.data_ptr(), t.numel(), _DT[t.dtype], peer, self._s()), "recv")
        return t

    def group_start(self):
        self._chk(self._L.lt_nccl_group_start(), "group_start")

    def group_end(self):
        self._chk(self._L.lt_nccl_group_end(), "group_end")

    def destroy(self):
        if self._c:
            self._L.lt_nccl_destroy(self._c)
            self._c = None


__all__ = ["NativeNccl", "NcclError", "nccl_version"]
