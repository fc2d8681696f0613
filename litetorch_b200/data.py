"""`lt.data`: Dataset, TensorDataset and the prefetching DataLoader
(src/bindings/python_bindings.cpp:886-915, src/data/dataloader.cpp:41-349).

`DataLoader(dataset, batch_size, shuffle, device, prefetch_limit)` keeps the reference methods `reset()`,
`next() -> (x, y) | None`, `save_state(path)`, `load_state(path)` (LTDL file).  For a `TensorDataset` the
batches are assembled by a native prefetch thread (csrc/runtime/dataloader.cpp) straight into pinned host
buffers and copied to the device asynchronously; a Python `Dataset` subclass (`size()/get(i)`) is
materialised once into a TensorDataset.
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, c_char_p, c_int, c_uint64, c_void_p
from typing import Optional, Tuple

import torch

from ._native import host_lib
from .core import Device, Tensor, _as_device, _unwrap


class Dataset:
    def size(self) -> int:
        raise NotImplementedError

    def get(self, index: int) -> Tuple[Tensor, Tensor]:
        raise NotImplementedError

    def __len__(self):
        return self.size()

    def __getitem__(self, index):
        return self.get(index)


class TensorDataset(Dataset):
    def __init__(self, x: Tensor, y: Tensor):
        self.x, self.y = x, y
        assert _unwrap(x).shape[0] == _unwrap(y).shape[0]

    def size(self) -> int:
        return _unwrap(self.x).shape[0]

    def get(self, index: int):
        return Tensor(_unwrap(self.x)[index]), Tensor(_unwrap(self.y)[index])


def _lib():
    lib = host_lib()
    if not getattr(lib, "_lt_dl_bound", False):
        lib.lt_dl_create.restype = c_void_p
        lib.lt_dl_create.argtypes = [c_void_p, c_void_p, c_uint64, c_uint64, c_uint64, c_uint64, c_int, c_uint64, c_int]
        lib.lt_dl_destroy.argtypes = [c_void_p]
        lib.lt_dl_reset.argtypes = [c_void_p]
        lib.lt_dl_next.argtypes = [c_void_p, c_void_p, c_void_p, POINTER(c_uint64)]
        lib.lt_dl_save_state.argtypes = [c_void_p, c_char_p]
        lib.lt_dl_load_state.argtypes = [c_void_p, c_char_p]
        lib.lt_dl_epoch.restype = c_uint64
        lib.lt_dl_epoch.argtypes = [c_void_p]
        lib.lt_dl_position.restype = c_uint64
        lib.lt_dl_position.argtypes = [c_void_p]
        lib._lt_dl_bound = True
    return lib


class DataLoader:
    def __init__(self, dataset: Dataset, batch_size: int = 32, shuffle: bool = False, device=None, prefetch_limit: int = 2,
                 seed: int = 0):
        if not isinstance(dataset, TensorDataset):
            xs, ys = zip(*[dataset.get(i) for i in range(dataset.size())])
            dataset = TensorDataset(Tensor(torch.stack([_unwrap(t) for t in xs])), Tensor(torch.stack([_unwrap(t) for t in ys])))
        self.dataset = dataset
        self.batch_size, self.shuffle = batch_size, shuffle
        self.device = _as_device(device)
        # the native loader reads from these two contiguous fp32 host arrays; keep them alive
        self._x = _unwrap(dataset.x).detach().to("cpu", torch.float32).contiguous()
        self._y = _unwrap(dataset.y).detach().to("cpu", torch.float32).contiguous()
        self._xshape, self._yshape = list(self._x.shape[1:]), list(self._y.shape[1:])
        n = self._x.shape[0]
        self._xs = max(1, self._x.numel() // max(n, 1))
        self._ys = max(1, self._y.numel() // max(n, 1))
        self._lib = _lib()
        self._h = self._lib.lt_dl_create(self._x.data_ptr(), self._y.data_ptr(), n, self._xs, self._ys, batch_size,
                                         1 if shuffle else 0, seed, prefetch_limit)
        pin = torch.cuda.is_available()
        self._bx = torch.empty(batch_size * self._xs, dtype=torch.float32, pin_memory=pin)
        self._by = torch.empty(batch_size * self._ys, dtype=torch.float32, pin_memory=pin)

    def __del__(self):
        try:
            self._lib.lt_dl_destroy(self._h)
        except Exception:
            pass

    def reset(self) -> None:
        self._lib.lt_dl_reset(self._h)

    def next(self) -> Optional[Tuple[Tensor, Tensor]]:
        cnt = c_uint64(0)
        if not self._lib.lt_dl_next(self._h, self._bx.data_ptr(), self._by.data_ptr(), ctypes.byref(cnt)):
            return None
        c = cnt.value
        x = self._bx[:c * self._xs].view(c, *self._xshape)
        y = self._by[:c * self._ys].view(c, *self._yshape)
        if self.device.type == "cuda":
            x, y = x.to(self.device, non_blocking=True), y.to(self.device, non_blocking=True)
            torch.cuda.current_stream().synchronize()  # the pinned staging buffers are reused by the next call
        else:
            x, y = x.clone(), y.clone()
        return Tensor(x), Tensor(y)

    def __iter__(self):
        while True:
            b = self.next()
            if b is None:
                return
            yield b

    @property
    def epoch(self) -> int:
        return int(self._lib.lt_dl_epoch(self._h))

    @property
    def position(self) -> int:
        return int(self._lib.lt_dl_position(self._h))

    def save_state(self, filepath: str) -> None:
        if self._lib.lt_dl_save_state(self._h, filepath.encode()) != 0:
            raise RuntimeError("failed to save dataloader state to %s" % filepath)

    def load_state(self, filepath: str) -> None:
        rc = self._lib.lt_dl_load_state(self._h, filepath.encode())
        if rc != 0:
            raise RuntimeError({-1: "cannot open %s", -2: "%s is malformed", -3: "CRC mismatch in %s",
                                -4: "%s was saved for a dataset of a different size"}.get(rc, "bad state file %s") % filepath)
