"""Checkpoint I/O (`lt.save / lt.load / save_parameters / load_parameters / save_optimizer_state /
load_optimizer_state`) in the reference's byte formats, written and read by the native runtime
(csrc/runtime/io.cpp).

* `LTW1`: magic, u32 count, per tensor {u32 ndims, i64 dims, u64 numel, f32 data}, CRC-32.  Tensors are
  positional (order of `module.parameters()`), always stored as fp32 (src/serialization/parameters.cpp:36-165).
* `LTAD` (Adam: i32 step, u32 n, n x m, n x v), `LTSG` (SGD velocities), `LTRP` (RMSprop square averages)
  (src/serialization/optimizer.cpp:37-393).  The reference cannot save AdamW (it throws); here AdamW and its
  variants use `LTAW`, an LTAD-shaped record, so that a resumed run continues bit-exactly.
* Loads validate magic, CRC, counts and every shape BEFORE any tensor is modified.
* `save_sharded / load_sharded`: one LTW1 file per rank plus a JSON manifest, for ZeRO-3 / TP / PP states.
"""
from __future__ import annotations

import ctypes
import json
import os
from ctypes import POINTER, c_char_p, c_float, c_int, c_int32, c_int64, c_uint32, c_uint64, c_uint8, c_void_p
from typing import List, Sequence

import torch

from ._native import host_lib
from .core import Tensor, _unwrap


class CheckpointError(RuntimeError):
    pass


def _lib():
    lib = host_lib()
    if not getattr(lib, "_lt_io_bound", False):
        lib.lt_ckpt_writer_open.restype = c_void_p
        lib.lt_ckpt_writer_open.argtypes = [c_char_p, c_char_p]
        lib.lt_ckpt_write_u32.argtypes = [c_void_p, c_uint32]
        lib.lt_ckpt_write_i32.argtypes = [c_void_p, c_int32]
        lib.lt_ckpt_write_u64.argtypes = [c_void_p, c_uint64]
        lib.lt_ckpt_write_tensor.argtypes = [c_void_p, c_int, POINTER(c_int64), c_void_p, c_uint64]
        lib.lt_ckpt_writer_close.argtypes = [c_void_p]
        lib.lt_ckpt_reader_open.restype = c_void_p
        lib.lt_ckpt_reader_open.argtypes = [c_char_p, ctypes.c_char * 4, POINTER(c_int)]
        lib.lt_ckpt_read_u32.argtypes = [c_void_p, POINTER(c_uint32)]
        lib.lt_ckpt_read_i32.argtypes = [c_void_p, POINTER(c_int32)]
        lib.lt_ckpt_read_tensor_header.argtypes = [c_void_p, POINTER(c_int), POINTER(c_int64), POINTER(c_uint64)]
        lib.lt_ckpt_read_tensor_data.argtypes = [c_void_p, c_void_p, c_uint64]
        lib.lt_ckpt_remaining.restype = c_uint64
        lib.lt_ckpt_remaining.argtypes = [c_void_p]
        lib.lt_ckpt_reader_close.argtypes = [c_void_p]
        lib._lt_io_bound = True
    return lib


def _write_tensor(lib, w, t: torch.Tensor):
    f = t.detach().to("cpu", torch.float32).contiguous()
    dims = (c_int64 * max(f.dim(), 1))(*f.shape)
    if lib.lt_ckpt_write_tensor(w, f.dim(), dims, f.data_ptr(), f.numel()) != 0:
        raise CheckpointError("write failure (disk full?)")


class _Reader:
    def __init__(self, path: str, expect: Sequence[bytes]):
        self.lib = _lib()
        magic = (ctypes.c_char * 4)()
        err = c_int(0)
        self.h = self.lib.lt_ckpt_reader_open(path.encode(), magic, ctypes.byref(err))
        if not self.h:
            raise CheckpointError({1: "cannot open %s", 2: "%s is truncated", 3: "CRC mismatch in %s"}.get(err.value, "bad file %s") % path)
        self.magic = bytes(magic)
        if self.magic not in expect:
            self.close()
            raise CheckpointError("%s: magic %r, expected one of %r" % (path, self.magic, list(expect)))

    def u32(self) -> int:
        v = c_uint32(0)
        if self.lib.lt_ckpt_read_u32(self.h, ctypes.byref(v)) != 0:
            raise CheckpointError("unexpected end of file")
        return v.value

    def i32(self) -> int:
        v = c_int32(0)
        if self.lib.lt_ckpt_read_i32(self.h, ctypes.byref(v)) != 0:
            raise CheckpointError("unexpected end of file")
        return v.value

    def tensor(self) -> torch.Tensor:
        nd, dims, numel = c_int(0), (c_int64 * 16)(), c_uint64(0)
        rc = self.lib.lt_ckpt_read_tensor_header(self.h, ctypes.byref(nd), dims, ctypes.byref(numel))
        if rc != 0:
            raise CheckpointError("malformed tensor record" if rc == -1 else "tensor record: numel does not match its dims")
        t = torch.empty([dims[i] for i in range(nd.value)], dtype=torch.float32)
        if self.lib.lt_ckpt_read_tensor_data(self.h, t.data_ptr(), numel.value) != 0:
            raise CheckpointError("unexpected end of file")
        return t

    def close(self):
        if self.h:
            self.lib.lt_ckpt_reader_close(self.h)
            self.h = None


def _params_of(obj) -> List[Tensor]:
    if hasattr(obj, "parameters"):
        return list(obj.parameters())
    return list(obj)


def save_parameters(params, filepath: str) -> None:
    lib = _lib()
    ps = _params_of(params)
    w = lib.lt_ckpt_writer_open(filepath.encode(), b"LTW1")
    if not w:
        raise CheckpointError("cannot open %s for writing" % filepath)
    lib.lt_ckpt_write_u32(w, len(ps))
    for p in ps:
        _write_tensor(lib, w, _unwrap(p))
    if lib.lt_ckpt_writer_close(w) != 0:
        raise CheckpointError("write failure while closing %s" % filepath)


def read_tensors(filepath: str) -> List[torch.Tensor]:
    r = _Reader(filepath, [b"LTW1"])
    try:
        return [r.tensor() for _ in range(r.u32())]
    finally:
        r.close()


def load_parameters(params, filepath: str) -> None:
    ps = _params_of(params)
    loaded = read_tensors(filepath)
    if len(loaded) != len(ps):
        raise CheckpointError("%s holds %d tensors, the model has %d" % (filepath, len(loaded), len(ps)))
    for i, (p, t) in enumerate(zip(ps, loaded)):
        if list(t.shape) != list(_unwrap(p).shape):
            raise CheckpointError("tensor %d: file shape %s, model shape %s" % (i, list(t.shape), list(_unwrap(p).shape)))
    for p, t in zip(ps, loaded):  # nothing was modified before every check passed
        with torch.no_grad():
            _unwrap(p).copy_(t.to(_unwrap(p).device, _unwrap(p).dtype))


def _opt_kind(opt):
    from . import optim as O
    if isinstance(opt, (O.AdamW, O.AdamW8bit, O.AdamWFP8, O.ZeRO3Optimizer)):
        return b"LTAW"
    if isinstance(opt, O.Adam):
        return b"LTAD"
    if isinstance(opt, O.SGD):
        return b"LTSG"
    if isinstance(opt, O.RMSprop):
        return b"LTRP"
    raise CheckpointError("unsupported optimizer type %s" % type(opt).__name__)


_MASTER_TRAILER = 0x5254534D          # "MSTR": optional record after the moments of an LTAD / LTAW file


def _state_target(p):
    """The tensor an optimizer state belongs to: the rank's shard for FSDP-sharded parameters, else the parameter."""
    shard = getattr(p, "shard", None)
    return _unwrap(shard) if shard is not None else _unwrap(p)


def _adam_states(opt):
    """(m, v) per parameter in the parameter's (or its shard's) shape; a state that does not exist on this rank
    (a replicated parameter of ZeRO3Optimizer that another rank owns, a parameter that never had a gradient) is
    written as an empty tensor."""
    from . import optim as O
    ms, vs = [], []
    none = torch.zeros(0)
    for i, p in enumerate(opt.params):
        if isinstance(opt, O.AdamW8bit):
            m = opt.m_q[i].float() * opt.m_scale[i] if opt.m_q[i] is not None else none
            v = opt.v_q[i].float() * opt.v_scale[i] if opt.v_q[i] is not None else none
        elif isinstance(opt, O.AdamWFP8):
            m = opt.m8[i].float() * opt.m_scale[i] if opt.m8[i] is not None else none
            v = opt.v8[i].float() * opt.v_scale[i] if opt.v8[i] is not None else none
        else:
            m = opt.m[i] if opt.m[i] is not None else none
            v = opt.v[i] if opt.v[i] is not None else none
        ms.append(m)
        vs.append(v)
    return ms, vs


def save_optimizer_state(optimizer, filepath: str) -> None:
    """SGD -> LTSG, RMSprop -> LTRP, Adam -> LTAD, AdamW family -> LTAW.  The Adam formats hold step count, m and v
    (the reference's layout, src/serialization/checkpoint.cpp) and, when the optimizer keeps fp32 master copies of
    low-precision parameters, those masters in a trailing record, so that a resumed bf16 run continues from the
    exact fp32 weights instead of their rounded copies."""
    opt = optimizer
    lib = _lib()
    kind = _opt_kind(opt)
    w = lib.lt_ckpt_writer_open(filepath.encode(), kind)
    if not w:
        raise CheckpointError("cannot open %s for writing" % filepath)
    n = len(opt.params)
    if kind in (b"LTAD", b"LTAW"):
        lib.lt_ckpt_write_i32(w, opt.step_count)
        lib.lt_ckpt_write_u32(w, n)
        ms, vs = _adam_states(opt)
        for t in ms + vs:
            _write_tensor(lib, w, t)
        masters = getattr(opt, "master", None)
        if masters is not None and any(m is not None for m in masters):
            lib.lt_ckpt_write_u32(w, _MASTER_TRAILER)
            lib.lt_ckpt_write_u32(w, n)
            for m in masters:
                _write_tensor(lib, w, m if m is not None else torch.zeros(0))
    else:
        lib.lt_ckpt_write_u32(w, n)
        states = opt.velocity if kind == b"LTSG" else opt.square_avg
        for p, s in zip(opt.params, states):
            _write_tensor(lib, w, s if s is not None else torch.zeros(_unwrap(p).shape))
    if lib.lt_ckpt_writer_close(w) != 0:
        raise CheckpointError("write failure while closing %s" % filepath)


def load_optimizer_state(optimizer, filepath: str) -> None:
    opt = optimizer
    from . import optim as O
    kind = _opt_kind(opt)
    r = _Reader(filepath, [kind])
    try:
        n_model = len(opt.params)
        if kind in (b"LTAD", b"LTAW"):
            step = r.i32()
            n = r.u32()
            if n != n_model:
                raise CheckpointError("%s holds %d states, the optimizer has %d parameters" % (filepath, n, n_model))
            ms = [r.tensor() for _ in range(n)]
            vs = [r.tensor() for _ in range(n)]
            masters = None
            try:
                tag = r.u32()
            except CheckpointError:
                tag = None                                  # a file without the master record (the reference's layout)
            if tag == _MASTER_TRAILER:
                if r.u32() != n:
                    raise CheckpointError("%s: master record count differs" % filepath)
                masters = [r.tensor() for _ in range(n)]
            for i, p in enumerate(opt.params):
                want = list(_state_target(p).shape)
                for t in (ms[i], vs[i]):
                    if t.numel() and list(t.shape) != want:
                        raise CheckpointError("state %d: shape %s differs from its parameter's %s" % (i, list(t.shape), want))
            opt.step_count = step
            for i, p in enumerate(opt.params):
                pt = _state_target(p)
                if ms[i].numel() == 0 and pt.numel() != 0:
                    continue                                # no state on this rank for this parameter
                if isinstance(opt, O.AdamW8bit):
                    opt.m_q[i], opt.m_scale[i] = opt._quant(ms[i].to(pt.device))
                    opt.v_q[i], opt.v_scale[i] = opt._quant(vs[i].to(pt.device))
                    opt._qstate[i] = None                   # the GPU kernel path re-imports codes and scales at its next step
                elif isinstance(opt, O.AdamWFP8):
                    opt.m8[i], opt.m_scale[i] = opt._store(ms[i].to(pt.device), opt.m_hist[i])
                    opt.v8[i], opt.v_scale[i] = opt._store(vs[i].to(pt.device), opt.v_hist[i])
                    opt._qstate[i] = None
                else:
                    opt._ensure_state(i, pt)
                    opt.m[i].copy_(ms[i])
                    opt.v[i].copy_(vs[i])
                    if masters is not None and masters[i].numel() and opt.master[i] is not None:
                        if list(masters[i].shape) != want_shape(pt):
                            raise CheckpointError("master %d: shape differs from its parameter" % i)
                        # Take the saved fp32 values; the next step keeps them wherever they round to the parameter
                        # as it is then (whether the parameters are loaded before or after this call) and falls back
                        # to the parameter's own value elsewhere.
                        opt.master[i].copy_(masters[i])
                        opt._pver[i] = None
        else:
            n = r.u32()
            if n != n_model:
                raise CheckpointError("%s holds %d states, the optimizer has %d parameters" % (filepath, n, n_model))
            ss = [r.tensor() for _ in range(n)]
            for i, p in enumerate(opt.params):
                if list(ss[i].shape) != list(_unwrap(p).shape):
                    raise CheckpointError("state %d: shape differs from its parameter" % i)
            tgt = opt.velocity if kind == b"LTSG" else opt.square_avg
            for i, p in enumerate(opt.params):
                tgt[i] = ss[i].to(_unwrap(p).device, torch.float32 if kind == b"LTRP" else _unwrap(p).dtype)
    finally:
        r.close()


def want_shape(t) -> list:
    return list(t.shape)


def save_optimizer_sharded(opt, directory: str, rank: int, world: int, tag: str = "optim") -> None:
    """One optimizer-state file per rank (shard-shaped states of ZeRO3Optimizer / FSDP) plus a manifest by rank 0."""
    os.makedirs(directory, exist_ok=True)
    save_optimizer_state(opt, os.path.join(directory, "%s.rank%05d.bin" % (tag, rank)))
    if rank == 0:
        man = {"format": "optimizer-sharded", "tag": tag, "world_size": world,
               "files": ["%s.rank%05d.bin" % (tag, r) for r in range(world)]}
        tmp = os.path.join(directory, "%s.manifest.json.tmp" % tag)
        with open(tmp, "w") as f:
            json.dump(man, f, indent=1)
        os.replace(tmp, os.path.join(directory, "%s.manifest.json" % tag))


def load_optimizer_sharded(opt, directory: str, rank: int, world: int, tag: str = "optim") -> None:
    with open(os.path.join(directory, "%s.manifest.json" % tag)) as f:
        man = json.load(f)
    if man["world_size"] != world:
        raise CheckpointError("optimizer state was written by %d ranks, this job has %d" % (man["world_size"], world))
    load_optimizer_state(opt, os.path.join(directory, man["files"][rank]))


def save(obj, filepath: str) -> None:
    from . import optim as O
    if isinstance(obj, O.Optimizer):
        save_optimizer_state(obj, filepath)
    else:
        save_parameters(obj, filepath)


def load(obj, filepath: str) -> None:
    from . import optim as O
    if isinstance(obj, O.Optimizer):
        load_optimizer_state(obj, filepath)
    else:
        load_parameters(obj, filepath)


# ------------------------------------------------------------------------------------------------ sharded checkpoints
def save_sharded(directory: str, tensors: Sequence[torch.Tensor], rank: int, world: int, tag: str = "model", meta=None) -> None:
    """Every rank writes its own LTW1 file; rank 0 also writes the manifest (JSON)."""
    os.makedirs(directory, exist_ok=True)
    save_parameters([Tensor(t) for t in tensors], os.path.join(directory, "%s.rank%05d.ltw1" % (tag, rank)))
    if rank == 0:
        man = {"format": "LTW1-sharded", "tag": tag, "world_size": world, "files": ["%s.rank%05d.ltw1" % (tag, r) for r in range(world)],
               "meta": meta or {}}
        tmp = os.path.join(directory, "%s.manifest.json.tmp" % tag)
        with open(tmp, "w") as f:
            json.dump(man, f, indent=1)
        os.replace(tmp, os.path.join(directory, "%s.manifest.json" % tag))


def load_sharded(directory: str, rank: int, world: int, tag: str = "model") -> List[torch.Tensor]:
    with open(os.path.join(directory, "%s.manifest.json" % tag)) as f:
        man = json.load(f)
    if man["world_size"] != world:
        raise CheckpointError("checkpoint was written by %d ranks, this job has %d" % (man["world_size"], world))
    return read_tensors(os.path.join(directory, man["files"][rank]))
