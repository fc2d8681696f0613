"""`lt.distributed.ProcessGroup` and the collective entry points of the reference API
(include/litetorch/distributed.h:29-92, src/bindings/python_bindings.cpp:724-791).

One process per GPU; `torch.distributed` is the plumbing (NCCL over NVLink for CUDA tensors, gloo for CPU
tensors - the reference's TCP star / POSIX-shm fallbacks map onto gloo).  The native TCP/file store
(csrc/runtime/store.cpp) provides rendezvous keys, heartbeats and a host-side barrier, so a dead rank is
noticed before the next collective instead of spinning forever (src/distributed/shm_ipc.cpp:188-192).

Semantics: `all_reduce` SUMS (as NCCL does; the reference's host fallbacks average - pass `average=True` for
that), `all_gather` concatenates rank-major, `reduce_scatter` sums.
"""
from __future__ import annotations

import ctypes
import os
import threading
import time
from ctypes import POINTER, c_char_p, c_int, c_int32, c_int64, c_uint64, c_void_p
from datetime import timedelta
from typing import List, Optional

import torch
import torch.distributed as dist

from .._native import host_lib
from ..core import Tensor, _unwrap


def _store_lib():
    lib = host_lib()
    if not getattr(lib, "_lt_store_bound", False):
        lib.lt_store_server_start.restype = c_void_p
        lib.lt_store_server_start.argtypes = [c_int, POINTER(c_int)]
        lib.lt_store_server_stop.argtypes = [c_void_p]
        lib.lt_store_connect.restype = c_void_p
        lib.lt_store_connect.argtypes = [c_char_p, c_int, c_int]
        lib.lt_store_close.argtypes = [c_void_p]
        lib.lt_store_set.argtypes = [c_void_p, c_char_p, c_void_p, c_uint64]
        lib.lt_store_get.restype = c_int64
        lib.lt_store_get.argtypes = [c_void_p, c_char_p, c_void_p, c_uint64, c_int]
        lib.lt_store_add.restype = c_int64
        lib.lt_store_add.argtypes = [c_void_p, c_char_p, c_int64]
        lib.lt_store_heartbeat.argtypes = [c_void_p, c_int]
        lib.lt_store_dead_ranks.argtypes = [c_void_p, c_int, POINTER(c_int32), c_int]
        lib.lt_store_barrier.argtypes = [c_void_p, c_char_p, c_int, c_int]
        lib.lt_store_silent_ranks.argtypes = [c_void_p, c_int, c_int, POINTER(c_int32), c_int]
        lib.lt_store_alive.argtypes = [c_void_p]
        lib.lt_store_set_timeout.argtypes = [c_void_p, c_int]
        lib.lt_filestore_set.argtypes = [c_char_p, c_char_p, c_void_p, c_uint64]
        lib.lt_filestore_get.restype = c_int64
        lib.lt_filestore_get.argtypes = [c_char_p, c_char_p, c_void_p, c_uint64, c_int]
        lib._lt_store_bound = True
    return lib


class RankFailure(RuntimeError):
    pass


class TCPStore:
    """Key-value rendezvous served by rank 0."""

    def __init__(self, host: str, port: int, is_server: bool, timeout_s: float = 60.0):
        self._lib = _store_lib()
        self._server = None
        self.port = port
        if is_server:
            p = c_int(0)
            self._server = self._lib.lt_store_server_start(port, ctypes.byref(p))
            if not self._server:
                raise RuntimeError("cannot bind the store to port %d" % port)
            self.port = p.value
        self._c = self._lib.lt_store_connect(host.encode(), self.port, int(timeout_s * 1000))
        if not self._c:
            raise RuntimeError("cannot reach the store at %s:%d within %.0f s" % (host, self.port, timeout_s))

    def set(self, key: str, value: bytes):
        if self._lib.lt_store_set(self._c, key.encode(), value, len(value)) != 0:
            raise RuntimeError("store set(%s) failed" % key)

    def get(self, key: str, timeout_s: float = 60.0) -> bytes:
        buf = ctypes.create_string_buffer(1 << 20)
        n = self._lib.lt_store_get(self._c, key.encode(), buf, 1 << 20, int(timeout_s * 1000))
        if n == -2:
            raise TimeoutError("key %r did not appear within %.1f s" % (key, timeout_s))
        if n < 0:
            raise RuntimeError("store get(%s) failed" % key)
        return buf.raw[:n]

    def add(self, key: str, delta: int) -> int:
        return int(self._lib.lt_store_add(self._c, key.encode(), delta))

    def barrier(self, key: str, world: int, timeout_s: float = 60.0):
        rc = self._lib.lt_store_barrier(self._c, key.encode(), world, int(timeout_s * 1000))
        if rc == -2:
            raise TimeoutError("barrier %r timed out after %.1f s" % (key, timeout_s))
        if rc != 0:
            raise RuntimeError("barrier %r failed" % key)

    def heartbeat(self, rank: int):
        self._lib.lt_store_heartbeat(self._c, rank)

    def dead_ranks(self, ttl_s: float) -> List[int]:
        out = (c_int32 * 1024)()
        n = self._lib.lt_store_dead_ranks(self._c, int(ttl_s * 1000), out, 1024)
        return [int(out[i]) for i in range(max(n, 0))]

    def silent_ranks(self, world: int, ttl_s: float) -> List[int]:
        """Ranks of [0, world) without any heartbeat so far, or with a last heartbeat older than `ttl_s`."""
        out = (c_int32 * max(world, 1))()
        n = self._lib.lt_store_silent_ranks(self._c, world, int(ttl_s * 1000), out, max(world, 1))
        if n < 0:
            raise RuntimeError("store connection lost")
        return [int(out[i]) for i in range(n)]

    def alive(self) -> bool:
        """False once an I/O error or a timeout has closed the connection (every later call fails at once)."""
        return bool(self._c) and self._lib.lt_store_alive(self._c) == 1

    def close(self):
        if self._c:
            self._lib.lt_store_close(self._c)
            self._c = None
        if self._server:
            self._lib.lt_store_server_stop(self._server)
            self._server = None


class FileStore:
    """The same operations over a shared directory (the reference's LITETORCH_RENDEZVOUS_FILE mechanism)."""

    def __init__(self, directory: str):
        self.dir = directory
        self._lib = _store_lib()

    def set(self, key: str, value: bytes):
        if self._lib.lt_filestore_set(self.dir.encode(), key.encode(), value, len(value)) != 0:
            raise RuntimeError("file store set(%s) failed" % key)

    def get(self, key: str, timeout_s: float = 60.0) -> bytes:
        buf = ctypes.create_string_buffer(1 << 20)
        n = self._lib.lt_filestore_get(self.dir.encode(), key.encode(), buf, 1 << 20, int(timeout_s * 1000))
        if n == -2:
            raise TimeoutError("key %r did not appear within %.1f s" % (key, timeout_s))
        return buf.raw[:n]


class Watchdog:
    """Background heartbeat; `check()` raises RankFailure when a peer's heartbeat is older than `ttl_s`."""

    def __init__(self, store: TCPStore, rank: int, interval_s: float = 0.5, ttl_s: float = 5.0,
                 world_size: Optional[int] = None, grace_s: float = 10.0):
        """world_size: when given, `check()` also reports ranks that never sent a heartbeat once `grace_s` seconds have
        passed since this watchdog started (a rank that died during start-up never shows up in the heartbeat table)."""
        self.store, self.rank, self.interval, self.ttl = store, rank, interval_s, ttl_s
        self.world_size, self.grace = world_size, grace_s
        self._t0 = time.monotonic()
        self._stop = threading.Event()
        self._t = threading.Thread(target=self._run, daemon=True)
        self._t.start()

    def _run(self):
        while not self._stop.is_set():
            try:
                self.store.heartbeat(self.rank)
            except Exception:
                return
            self._stop.wait(self.interval)

    def check(self):
        if self.world_size is not None and time.monotonic() - self._t0 >= self.grace:
            dead = [r for r in self.store.silent_ranks(self.world_size, self.ttl) if r != self.rank]
        else:
            dead = [r for r in self.store.dead_ranks(self.ttl) if r != self.rank]
        if dead:
            raise RankFailure("ranks %s stopped sending heartbeats (ttl %.1f s)" % (dead, self.ttl))

    def stop(self):
        self._stop.set()
        self._t.join(timeout=2)


class ProcessGroup:
    _inst = None

    def __init__(self):
        self.rank, self.world_size = 0, 1
        self._initialized = False
        self.store: Optional[TCPStore] = None
        self.watchdog: Optional[Watchdog] = None

    @staticmethod
    def get() -> "ProcessGroup":
        if ProcessGroup._inst is None:
            ProcessGroup._inst = ProcessGroup()
        return ProcessGroup._inst

    def init(self, rank: int, world_size: int, master_addr: str = "127.0.0.1", master_port: int = 29500,
             backend: Optional[str] = None, timeout_s: float = 600.0, with_store: bool = False) -> None:
        self.rank, self.world_size = rank, world_size
        if not dist.is_initialized():
            if backend is None:
                backend = "nccl" if torch.cuda.is_available() else "gloo"
            kw = {}
            if backend == "nccl":
                local = int(os.environ.get("LOCAL_RANK", rank % max(torch.cuda.device_count(), 1)))
                torch.cuda.set_device(local)
                kw["device_id"] = torch.device("cuda", local)
            # The reference publishes its communicator id through a file named by LITETORCH_RENDEZVOUS_FILE (or
            # NCCL_UNIQUE_ID_FILE; src/distributed/distributed.cpp:824-850); here the same variable selects
            # torch.distributed's file rendezvous instead of the TCP one.
            rend = rendezvous_file()
            method = ("file://" + os.path.abspath(rend)) if rend else "tcp://%s:%d" % (master_addr, master_port)
            dist.init_process_group(backend, init_method=method, rank=rank,
                                    world_size=world_size, timeout=timedelta(seconds=timeout_s), **kw)
        if with_store:
            self.store = TCPStore(master_addr, master_port + 1, is_server=(rank == 0))
            self.watchdog = Watchdog(self.store, rank, world_size=world_size)
        self._initialized = True

    def shutdown(self) -> None:
        if self.watchdog:
            self.watchdog.stop()
            self.watchdog = None
        if self.store:
            self.store.close()
            self.store = None
        if dist.is_initialized():
            dist.destroy_process_group()
        self._initialized = False

    def is_initialized(self) -> bool:
        return self._initialized or dist.is_initialized()

    def get_rank(self) -> int:
        return dist.get_rank() if dist.is_initialized() else self.rank

    def get_world_size(self) -> int:
        return dist.get_world_size() if dist.is_initialized() else self.world_size

    def _live(self) -> bool:
        if self.watchdog:
            self.watchdog.check()
        return dist.is_initialized() and dist.get_world_size() > 1

    def all_reduce(self, tensor: Tensor, average: bool = False) -> Tensor:
        t = _unwrap(tensor)
        if self._live():
            with torch.no_grad():
                dist.all_reduce(t)
                if average:
                    t.div_(dist.get_world_size())
        return tensor

    def broadcast(self, tensor: Tensor, src: int = 0) -> Tensor:
        if self._live():
            with torch.no_grad():
                dist.broadcast(_unwrap(tensor), src)
        return tensor

    def all_gather(self, shard: Tensor, full: Optional[Tensor] = None) -> Tensor:
        s = _unwrap(shard).contiguous()
        W = self.get_world_size()
        out = _unwrap(full) if full is not None else torch.empty((W * s.shape[0],) + tuple(s.shape[1:]), dtype=s.dtype, device=s.device)
        if self._live():
            dist.all_gather_into_tensor(out.view(-1), s.view(-1))
        else:
            out.view(-1)[:s.numel()].copy_(s.view(-1))
        return full if full is not None else Tensor(out)

    def reduce_scatter(self, shard: Tensor, full: Optional[Tensor] = None) -> Tensor:
        """`reduce_scatter(shard, full)`, the reference's form (src/bindings/python_bindings.cpp:733), sums `full` over the
        ranks and leaves this rank's slice in `shard`; `reduce_scatter(full)` returns the slice as a new tensor."""
        if full is None:
            shard, full = None, shard
        f = _unwrap(full).contiguous()
        W = self.get_world_size()
        out = _unwrap(shard) if shard is not None else torch.empty(f.numel() // W, dtype=f.dtype, device=f.device)
        if self._live():
            if f.is_cuda:
                dist.reduce_scatter_tensor(out.view(-1), f.view(-1))
            else:  # gloo has no reduce_scatter: all-reduce then slice
                tmp = f.clone()
                dist.all_reduce(tmp)
                out.view(-1).copy_(tmp.view(W, -1)[dist.get_rank()])
        else:
            out.view(-1).copy_(f.view(-1)[:out.numel()])
        return shard if shard is not None else Tensor(out)

    def send_tensor(self, tensor: Tensor, dst: int) -> None:
        """Shape-carrying send: a small header (ndim, dtype code, dims) precedes the payload, as the reference's wire
        format does (src/distributed/distributed.cpp:577-748), so the receiver needs no prior shape."""
        t = _unwrap(tensor).contiguous()
        hdr = torch.zeros(10, dtype=torch.int64)
        hdr[0] = t.dim()
        hdr[1] = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2, torch.int64: 3}.get(t.dtype, 0)
        for i, d in enumerate(t.shape):
            hdr[2 + i] = d
        dist.send(hdr.to(t.device) if t.is_cuda else hdr, dst)
        dist.send(t, dst)

    def recv_tensor(self, tensor=None, src: Optional[int] = None, device=None) -> Tensor:
        """`recv_tensor(src)` returns the tensor rank `src` sent with `send_tensor` (shape and dtype travel with it);
        `recv_tensor(tensor, src)`, the reference's form (src/bindings/python_bindings.cpp:735), also copies it into `tensor`."""
        from ..core import _as_device
        dst = None
        if isinstance(tensor, Tensor) or torch.is_tensor(tensor):
            dst = tensor
        elif tensor is not None and src is None:
            src = int(tensor)
        if src is None:
            raise TypeError("recv_tensor needs the source rank")
        if dst is not None and device is None:
            device = _unwrap(dst).device
        dev = _as_device(device) if device is not None else (torch.device("cuda", torch.cuda.current_device())
                                                             if dist.get_backend() == "nccl" else torch.device("cpu"))
        hdr = torch.zeros(10, dtype=torch.int64, device=dev)
        dist.recv(hdr, src)
        h = hdr.tolist()
        dtype = {0: torch.float32, 1: torch.bfloat16, 2: torch.float16, 3: torch.int64}[int(h[1])]
        t = torch.empty([int(x) for x in h[2:2 + int(h[0])]], dtype=dtype, device=dev)
        dist.recv(t, src)
        if dst is not None:
            d = _unwrap(dst)
            with torch.no_grad():
                if d.numel() == t.numel() and d.dtype == t.dtype:
                    d.copy_(t.reshape(d.shape))
                else:                       # the destination takes the sender's shape, as the reference's does
                    d.data = t.to(d.dtype)
            return dst if isinstance(dst, Tensor) else Tensor(dst)
        return Tensor(t)

    def sync_comm(self) -> None:
        if torch.cuda.is_available():
            torch.cuda.synchronize()

    def barrier(self, timeout_s: float = 600.0) -> None:
        if self.store is not None:
            self.store.barrier("pg_barrier", self.get_world_size(), timeout_s)
        elif self._live():
            dist.barrier()


def rendezvous_file() -> Optional[str]:
    """The path named by LITETORCH_RENDEZVOUS_FILE or NCCL_UNIQUE_ID_FILE, or None."""
    for k in ("LITETORCH_RENDEZVOUS_FILE", "NCCL_UNIQUE_ID_FILE"):
        v = os.environ.get(k, "")
        if v:
            return v
    return None


def init_process_group(rank: int, world_size: int, master_addr: str = "127.0.0.1", master_port: int = 29500, **kw) -> ProcessGroup:
    pg = ProcessGroup.get()
    pg.init(rank, world_size, master_addr, master_port, **kw)
    return pg


# Free functions over the process-wide group, as in the reference's C++ API (include/litetorch/distributed.h:82-92).
def shutdown() -> None:
    ProcessGroup.get().shutdown()


def get_rank() -> int:
    return ProcessGroup.get().get_rank()


def get_world_size() -> int:
    return ProcessGroup.get().get_world_size()


def barrier(timeout_s: float = 600.0) -> None:
    ProcessGroup.get().barrier(timeout_s)


def all_reduce(tensor: Tensor, average: bool = False) -> Tensor:
    return ProcessGroup.get().all_reduce(tensor, average)


def all_reduce_async(tensor: Tensor):
    """Starts the sum and returns a handle whose `wait()` (or `get()`) completes it."""
    class _Done:
        def __init__(self, work):
            self.work = work

        def wait(self):
            if self.work is not None:
                self.work.wait()
                self.work = None

        get = wait
    pg = ProcessGroup.get()
    return _Done(dist.all_reduce(_unwrap(tensor), async_op=True) if pg._live() else None)


def broadcast(tensor: Tensor, src: int = 0) -> Tensor:
    return ProcessGroup.get().broadcast(tensor, src)


def all_gather(shard: Tensor, full: Optional[Tensor] = None) -> Tensor:
    return ProcessGroup.get().all_gather(shard, full)


def reduce_scatter(shard: Tensor, full: Optional[Tensor] = None) -> Tensor:
    return ProcessGroup.get().reduce_scatter(shard, full)


def send_tensor(tensor: Tensor, dst: int) -> None:
    ProcessGroup.get().send_tensor(tensor, dst)


def recv_tensor(tensor=None, src: Optional[int] = None, device=None) -> Tensor:
    return ProcessGroup.get().recv_tensor(tensor, src, device)


def all_reduce_grads(module, average: bool = True) -> None:
    """All-reduce every parameter gradient of a module (src/distributed/distributed.cpp:755-765)."""
    all_reduce_bucketed([p.grad for p in module.parameters() if p.grad is not None], average=average)


def all_reduce_bucketed(tensors, bucket_bytes: int = 25 * 1024 * 1024, average: bool = False) -> None:
    """Flatten tensors into buckets of at most `bucket_bytes`, all-reduce each bucket once, scatter the results back
    (src/distributed/distributed.cpp:1204-1284)."""
    if not (dist.is_initialized() and dist.get_world_size() > 1):
        return
    ts = [_unwrap(t) for t in tensors]
    bucket, size = [], 0

    def flush():
        nonlocal bucket, size
        if not bucket:
            return
        flat = torch.cat([b.reshape(-1) for b in bucket])
        dist.all_reduce(flat)
        if average:
            flat.div_(dist.get_world_size())
        off = 0
        for b in bucket:
            b.copy_(flat[off:off + b.numel()].view_as(b))
            off += b.numel()
        bucket, size = [], 0
    with torch.no_grad():
        for t in ts:
            nb = t.numel() * t.element_size()
            if size + nb > bucket_bytes and bucket:
                flush()
            bucket.append(t)
            size += nb
        flush()


class OverlappedAllReducer:
    """Reductions issued on a communication stream while compute continues; `sync()` makes the compute stream wait
    for them (the reference's version waits on the wrong stream: src/distributed/distributed.cpp:1184-1190)."""

    _inst = None

    def __init__(self):
        self._works = []
        self._stream = None

    @staticmethod
    def get() -> "OverlappedAllReducer":
        if OverlappedAllReducer._inst is None:
            OverlappedAllReducer._inst = OverlappedAllReducer()
        return OverlappedAllReducer._inst

    def push_and_all_reduce(self, tensor: Tensor) -> None:
        if dist.is_initialized() and dist.get_world_size() > 1:
            self._works.append(dist.all_reduce(_unwrap(tensor), async_op=True))

    def push_and_reduce_scatter(self, shard: Tensor, full: Tensor) -> None:
        if dist.is_initialized() and dist.get_world_size() > 1 and _unwrap(full).is_cuda:
            self._works.append(dist.reduce_scatter_tensor(_unwrap(shard).view(-1), _unwrap(full).contiguous().view(-1), async_op=True))
        else:
            ProcessGroup.get().reduce_scatter(shard, full)

    def sync(self) -> None:
        for w in self._works:
            w.wait()
        self._works.clear()


def overlapped_all_reduce(tensor: Tensor) -> None:
    OverlappedAllReducer.get().push_and_all_reduce(tensor)


def overlapped_reduce_scatter(shard: Tensor, full: Tensor) -> None:
    OverlappedAllReducer.get().push_and_reduce_scatter(shard, full)


def sync_overlapped_all_reduce() -> None:
    OverlappedAllReducer.get().sync()
