"""`lt.memory`: device residency under a byte limit - evict to host, swap back in, LRU order, pins.

The reference keeps every storage registered with a MemoryManager that, when a new allocation would exceed the
limit (512 MB by default there), evicts the least-recently-used idle storages to host memory and swaps them back in
on their next use (src/tensor/storage.cpp:124-205, src/memory_manager/memory_manager.cpp:54-107, StorageUseGuard pins:
src/tensor/tensor_core.cpp:17-33).  Here residency is opt-in (180 GB of HBM3e are there to be used): a
`ResidencyManager(limit_bytes)` manages the tensors registered with it - typically optimizer state or saved
activations of a model that does not fit - on top of the native LRU list (`lt_lru_*` in csrc/runtime/allocator.cpp),
which decides who leaves; this module moves the bytes (pinned host buffers, `non_blocking` copies on the current stream).

    mm = lt.memory.ResidencyManager(limit_bytes=2 << 20, device="cuda")
    h = mm.register(tensor)          # may evict others to make room
    with mm.use(h) as t:             # swapped in if needed, pinned (not evictable) inside the block
        ...
"""
from __future__ import annotations

import contextlib
import ctypes
from typing import Dict, Optional

import torch

from ._native import host_lib


def _lib():
    L = host_lib()
    if not getattr(L, "_lt_lru_bound", False):
        L.lt_lru_create.restype = ctypes.c_void_p
        L.lt_lru_create.argtypes = [ctypes.c_uint64, ctypes.c_void_p, ctypes.c_void_p]
        L.lt_lru_destroy.argtypes = [ctypes.c_void_p]
        L.lt_lru_register.argtypes = [ctypes.c_void_p, ctypes.c_uint64, ctypes.c_uint64, ctypes.POINTER(ctypes.c_uint64), ctypes.c_int]
        L.lt_lru_unregister.argtypes = [ctypes.c_void_p, ctypes.c_uint64]
        L.lt_lru_touch.argtypes = [ctypes.c_void_p, ctypes.c_uint64]
        L.lt_lru_pin.argtypes = [ctypes.c_void_p, ctypes.c_uint64, ctypes.c_int]
        L.lt_lru_used.restype = ctypes.c_uint64
        L.lt_lru_used.argtypes = [ctypes.c_void_p]
        L.lt_lru_evictions.restype = ctypes.c_uint64
        L.lt_lru_evictions.argtypes = [ctypes.c_void_p]
        L.lt_lru_set_limit.argtypes = [ctypes.c_void_p, ctypes.c_uint64]
        L._lt_lru_bound = True
    return L


class Handle:
    """One managed tensor: `tensor` is the device copy while resident, `host` the pinned copy while evicted."""
    __slots__ = ("id", "tensor", "host", "bytes", "shape", "dtype", "pins")

    def __init__(self, hid: int, t: torch.Tensor):
        self.id, self.tensor, self.host = hid, t, None
        self.bytes = t.numel() * t.element_size()
        self.shape, self.dtype, self.pins = tuple(t.shape), t.dtype, 0

    @property
    def resident(self) -> bool:
        return self.tensor is not None


class ResidencyManager:
    def __init__(self, limit_bytes: int, device="cuda"):
        self.device = torch.device(device)
        self._L = _lib()
        self._h = self._L.lt_lru_create(int(limit_bytes), None, None)
        self._items: Dict[int, Handle] = {}
        self._next = 1
        self.swap_ins = 0

    def __del__(self):
        try:
            self._L.lt_lru_destroy(self._h)
        except Exception:
            pass

    # ---- bookkeeping
    @property
    def resident_bytes(self) -> int:
        return int(self._L.lt_lru_used(self._h))

    @property
    def evictions(self) -> int:
        return int(self._L.lt_lru_evictions(self._h))

    def set_limit(self, limit_bytes: int) -> None:
        self._L.lt_lru_set_limit(self._h, int(limit_bytes))

    def _admit(self, h: Handle) -> None:
        """Tell the LRU list that `h` is (again) resident; move whoever it pushes out to the host."""
        out = (ctypes.c_uint64 * 256)()
        n = self._L.lt_lru_register(self._h, h.id, h.bytes, out, 256)
        for i in range(min(n, 256)):
            self._evict(self._items[int(out[i])])

    def _evict(self, v: Handle) -> None:
        if v.tensor is None:
            return
        pin = self.device.type == "cuda"
        if v.host is None:
            v.host = torch.empty(v.shape, dtype=v.dtype, pin_memory=pin)
        v.host.copy_(v.tensor, non_blocking=pin)
        if pin:
            # the device block may be handed out again as soon as it is freed: make the copy's stream own the order
            v.tensor.record_stream(torch.cuda.current_stream())
        v.tensor = None

    # ---- public
    def register(self, t: torch.Tensor) -> Handle:
        """Take over a tensor that lives on the managed device.  The caller should drop its own reference: the
        handle's `tensor` is the only one that keeps the device memory alive, so that eviction really frees it."""
        h = Handle(self._next, t)
        self._next += 1
        self._items[h.id] = h
        self._admit(h)
        return h

    def release(self, h: Handle) -> None:
        self._L.lt_lru_unregister(self._h, h.id)
        self._items.pop(h.id, None)
        h.tensor = h.host = None

    def fetch(self, h: Handle) -> torch.Tensor:
        """The device tensor of `h`, swapped in (and others evicted to make room) when it had been moved out."""
        if h.tensor is None:
            pin = self.device.type == "cuda"
            h.pins += 1                                   # a storage being brought in is never its own victim
            try:
                h.tensor = torch.empty(h.shape, dtype=h.dtype, device=self.device)
                self._admit(h)
                h.tensor.copy_(h.host, non_blocking=pin)
                self.swap_ins += 1
            finally:
                h.pins -= 1
        else:
            self._L.lt_lru_touch(self._h, h.id)
        return h.tensor

    @contextlib.contextmanager
    def use(self, h: Handle):
        """`with mm.use(h) as t:` - resident and not evictable inside the block (the reference's StorageUseGuard)."""
        t = self.fetch(h)
        h.pins += 1
        self._L.lt_lru_pin(self._h, h.id, 1)
        try:
            yield t
        finally:
            h.pins -= 1
            if h.pins == 0:
                self._L.lt_lru_pin(self._h, h.id, 0)


__all__ = ["ResidencyManager", "Handle"]
