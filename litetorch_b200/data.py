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


class TokenStream:
    """Batches of `[batch_size, seq_len]` inputs and next-token targets from a flat binary file of token ids (uint16 or
    uint32), for language-model training.  The file is memory-mapped by the native runtime (csrc/runtime/tokenstream.cpp):
    windows of `seq_len + 1` tokens are permuted per epoch from `(seed, epoch)`, dealt to the ranks round-robin (disjoint
    windows, the same number of batches on every rank) and widened to int64 by a prefetch thread into pinned buffers.

    `next()` returns `(tokens, targets)` as CPU tensors in pinned memory - what `Trainer.step` takes - or None at the end of
    an epoch (`next_epoch()` goes on; iterating the object does so by itself).  The buffers rotate over `prefetch_limit + 1`
    slots: a batch stays valid until that many further batches have been taken.  The position is `(epoch, position)` and
    nothing else: `save_state / load_state` (or `state_dict / load_state_dict`) resume with exactly the batches the
    interrupted job would have seen, so a `TokenStream` can be the `loader=` of `Trainer.save / load`."""

    def __init__(self, path: str, seq_len: int, batch_size: int, dtype: str = "uint16", shuffle: bool = True, seed: int = 0,
                 rank: Optional[int] = None, world: Optional[int] = None, prefetch_limit: int = 2):
        import os
        self._lib = _ts_lib()
        self.path, self.seq_len, self.batch_size = path, int(seq_len), int(batch_size)
        self.rank = int(os.environ.get("RANK", "0")) if rank is None else int(rank)
        self.world = int(os.environ.get("WORLD_SIZE", "1")) if world is None else int(world)
        nbytes = {"uint16": 2, "uint32": 4}[dtype]
        self._h = self._lib.lt_ts_open(path.encode(), nbytes, self.seq_len, self.batch_size, 1 if shuffle else 0, int(seed),
                                       self.rank, self.world, int(prefetch_limit))
        if not self._h:
            raise RuntimeError("cannot open %s as a token stream of %s (a batch needs %d windows of %d + 1 tokens)"
                               % (path, dtype, self.batch_size * self.world, self.seq_len))
        pin = torch.cuda.is_available()
        self._slots = [(torch.empty(batch_size, seq_len, dtype=torch.int64, pin_memory=pin),
                        torch.empty(batch_size, seq_len, dtype=torch.int64, pin_memory=pin)) for _ in range(prefetch_limit + 1)]
        self._turn = 0

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            try:
                self._lib.lt_ts_close(h)
            except Exception:
                pass

    num_tokens = property(lambda self: int(self._lib.lt_ts_num_tokens(self._h)))
    num_windows = property(lambda self: int(self._lib.lt_ts_num_windows(self._h)))
    batches_per_epoch = property(lambda self: int(self._lib.lt_ts_batches_per_epoch(self._h)))
    epoch = property(lambda self: int(self._lib.lt_ts_epoch(self._h)))
    position = property(lambda self: int(self._lib.lt_ts_position(self._h)))

    def next(self) -> Optional[Tuple[torch.Tensor, torch.Tensor]]:
        tok, tgt = self._slots[self._turn]
        if not self._lib.lt_ts_next(self._h, tok.data_ptr(), tgt.data_ptr()):
            return None
        self._turn = (self._turn + 1) % len(self._slots)
        return tok, tgt

    def next_epoch(self) -> None:
        self._lib.lt_ts_next_epoch(self._h)

    reset = next_epoch          # the DataLoader's name for "start the next epoch"

    def __iter__(self):
        """Endless: batches of this epoch, then of the next ones."""
        while True:
            b = self.next()
            if b is None:
                self.next_epoch()
                continue
            yield b

    def state_dict(self) -> dict:
        return {"epoch": self.epoch, "position": self.position, "seq_len": self.seq_len, "batch_size": self.batch_size,
                "world": self.world, "num_tokens": self.num_tokens}

    def load_state_dict(self, state: dict) -> None:
        for k in ("seq_len", "batch_size", "world", "num_tokens"):
            if int(state[k]) != getattr(self, k):
                raise RuntimeError("token stream state was saved with %s = %s, this stream has %s" % (k, state[k], getattr(self, k)))
        self._lib.lt_ts_seek(self._h, int(state["epoch"]), int(state["position"]))

    def save_state(self, filepath: str) -> None:
        import json
        import os
        with open(filepath + ".tmp", "w") as f:
            json.dump(self.state_dict(), f)
        os.replace(filepath + ".tmp", filepath)

    def load_state(self, filepath: str) -> None:
        import json
        with open(filepath) as f:
            self.load_state_dict(json.load(f))


def _ts_lib():
    lib = host_lib()
    if not getattr(lib, "_lt_ts_bound", False):
        from ctypes import c_int64
        lib.lt_ts_open.restype = c_void_p
        lib.lt_ts_open.argtypes = [c_char_p, c_int, c_uint64, c_uint64, c_int, c_uint64, c_int, c_int, c_int]
        lib.lt_ts_close.argtypes = [c_void_p]
        for fn in ("lt_ts_num_tokens", "lt_ts_num_windows", "lt_ts_batches_per_epoch", "lt_ts_epoch", "lt_ts_position"):
            getattr(lib, fn).restype = c_uint64
            getattr(lib, fn).argtypes = [c_void_p]
        lib.lt_ts_next.argtypes = [c_void_p, c_void_p, c_void_p]
        lib.lt_ts_next_epoch.argtypes = [c_void_p]
        lib.lt_ts_seek.argtypes = [c_void_p, c_uint64, c_uint64]
        lib._lt_ts_bound = True
    return lib


def pack_examples(examples, seq_len: int, pad_id: int = 0, mask_prompt: bool = True):
    """Supervised fine-tuning batches from `(prompt_ids, response_ids)` pairs: examples are laid end to end into rows of
    `seq_len + 1` tokens (a new row starts when the next example does not fit; an example longer than a row is cut), and
    the targets are -100 - ignored by the engine's loss - on prompt tokens (unless `mask_prompt=False`), on padding, and
    where a row's next token belongs to another example.  Returns `(tokens [rows, seq_len], targets [rows, seq_len])` as
    int64 CPU tensors, ready for `Trainer.step`."""
    rows_t, rows_m = [], []
    cur_t, cur_m = [], []

    def flush():
        if cur_t:
            pad = seq_len + 1 - len(cur_t)
            rows_t.append(cur_t + [pad_id] * pad)
            rows_m.append(cur_m + [False] * pad)

    for prompt, response in examples:
        toks = [int(t) for t in prompt] + [int(t) for t in response]
        keep = [not mask_prompt] * len(prompt) + [True] * len(response)
        toks, keep = toks[:seq_len + 1], keep[:seq_len + 1]
        if len(cur_t) + len(toks) > seq_len + 1:
            flush()
            cur_t, cur_m = [], []
        if cur_t:
            keep = [False] + keep[1:]            # the first token of an example is never predicted from the previous one
        cur_t, cur_m = cur_t + toks, cur_m + keep
    flush()
    if not rows_t:
        raise ValueError("no examples")
    t = torch.tensor(rows_t, dtype=torch.int64)
    m = torch.tensor(rows_m, dtype=torch.bool)
    tokens, targets = t[:, :-1].contiguous(), t[:, 1:].clone()
    targets[~m[:, 1:]] = -100                    # position j predicts token j + 1: masked when that token is not kept
    return tokens, targets
