"""Tensor, Device and DataType of the public API.

`lt.Tensor` is a thin handle over a `torch.Tensor` (PyTorch is the tensor/autograd layer of this build);
it keeps the method names of the reference binding (src/bindings/python_bindings.cpp:226-256): `create,
from_vector, zeros, shape, strides, dtype, device, requires_grad, grad, numel, item, to_vector,
backward(gradient, create_graph), zero_grad, to, view, reshape, transpose, contiguous, is_contiguous,
clone, cast, copy_, add_, register_hook`.  Index tensors may be float tensors holding integers, as in the
reference (Embedding, cross-entropy targets, block tables).
"""
from __future__ import annotations

import enum
import os
from typing import Callable, List, Optional, Sequence, Union

import torch


class DeviceType(enum.IntEnum):
    CPU = 0
    GPU = 1
    META = 2
    TPU = 3   # kept for API compatibility; no such backend exists in this build


class Device:
    """Device(type, index) or Device("cuda:0" | "gpu" | "cpu" | "meta")."""

    def __init__(self, type: Union[DeviceType, str] = DeviceType.CPU, index: int = 0):
        if isinstance(type, str):
            s = type.lower()
            name, _, idx = s.partition(":")
            index = int(idx) if idx else 0
            if name in ("cuda", "gpu"):
                type = DeviceType.GPU
            elif name == "cpu":
                type = DeviceType.CPU
            elif name == "meta":
                type = DeviceType.META
            elif name == "tpu":
                raise ValueError("the TPU backend of the reference is not part of this build")
            else:
                raise ValueError("unknown device string %r" % type)
        self.type = DeviceType(type)
        self.index = int(index)

    def torch(self) -> torch.device:
        if self.type == DeviceType.GPU:
            return torch.device("cuda", self.index)
        if self.type == DeviceType.META:
            return torch.device("meta")
        return torch.device("cpu")

    @staticmethod
    def from_torch(d: torch.device) -> "Device":
        if d.type == "cuda":
            return Device(DeviceType.GPU, d.index or 0)
        if d.type == "meta":
            return Device(DeviceType.META, 0)
        return Device(DeviceType.CPU, 0)

    def to_string(self) -> str:
        return {DeviceType.CPU: "cpu", DeviceType.GPU: "cuda:%d" % self.index, DeviceType.META: "meta",
                DeviceType.TPU: "tpu:%d" % self.index}[self.type]

    __repr__ = to_string

    def __eq__(self, o):
        return isinstance(o, Device) and o.type == self.type and (o.index == self.index or self.type != DeviceType.GPU)

    def __hash__(self):
        return hash((int(self.type), self.index))


class DataType(enum.IntEnum):
    FP64 = 0
    FP32 = 1
    FP16 = 2
    BF16 = 3
    INT16 = 4
    INT8 = 5
    INT4 = 6
    NF4 = 7
    FP8_E4M3 = 8
    FP8_E5M2 = 9
    FP4_E2M1 = 10


DataType.FP4 = DataType.FP4_E2M1

_TO_TORCH = {
    DataType.FP64: torch.float64, DataType.FP32: torch.float32, DataType.FP16: torch.float16, DataType.BF16: torch.bfloat16,
    DataType.INT16: torch.int16, DataType.INT8: torch.int8, DataType.FP8_E4M3: torch.float8_e4m3fn,
    DataType.FP8_E5M2: torch.float8_e5m2,
}
_FROM_TORCH = {v: k for k, v in _TO_TORCH.items()}


def _as_device(d) -> torch.device:
    if isinstance(d, Device):
        return d.torch()
    if isinstance(d, str):
        return Device(d).torch()
    if d is None:
        return torch.device("cpu")
    return torch.device(d)


def _unwrap(x):
    return x._t if isinstance(x, Tensor) else x


class Tensor:
    __slots__ = ("_t", "_dtype_tag", "shard", "__weakref__")   # `shard`: this rank's slice under FSDP (as in the reference Tensor)

    def __init__(self, t: torch.Tensor, dtype_tag: Optional[DataType] = None):
        self._t = t
        self._dtype_tag = dtype_tag  # 4-bit formats are stored one code per int8/uint8 element, as in the reference

    # ---- construction
    @staticmethod
    def create(shape: Sequence[int], device=None, requires_grad: bool = False, dtype: DataType = DataType.FP32) -> "Tensor":
        t = torch.empty(list(shape), dtype=_TO_TORCH.get(dtype, torch.float32), device=_as_device(device))
        if requires_grad:
            t.requires_grad_(True)
        return Tensor(t)

    @staticmethod
    def from_vector(data, shape: Sequence[int], device=None, requires_grad: bool = False, dtype: DataType = DataType.FP32) -> "Tensor":
        t = torch.tensor(data, dtype=torch.float32).reshape(list(shape))
        td = _TO_TORCH.get(dtype, torch.float32)
        t = t.to(device=_as_device(device), dtype=td)
        if requires_grad:
            t.requires_grad_(True)
        return Tensor(t)

    @staticmethod
    def zeros(shape: Sequence[int], device=None, requires_grad: bool = False) -> "Tensor":
        t = torch.zeros(list(shape), dtype=torch.float32, device=_as_device(device))
        if requires_grad:
            t.requires_grad_(True)
        return Tensor(t)

    @staticmethod
    def from_torch(t: torch.Tensor) -> "Tensor":
        return Tensor(t)

    def torch(self) -> torch.Tensor:
        return self._t

    # ---- metadata
    @property
    def shape(self) -> List[int]:
        return list(self._t.shape)

    @property
    def strides(self) -> List[int]:
        return list(self._t.stride())

    @property
    def dtype(self) -> DataType:
        return self._dtype_tag if self._dtype_tag is not None else _FROM_TORCH.get(self._t.dtype, DataType.FP32)

    @property
    def device(self) -> Device:
        return Device.from_torch(self._t.device)

    @property
    def requires_grad(self) -> bool:
        return self._t.requires_grad

    @requires_grad.setter
    def requires_grad(self, v: bool):
        self._t.requires_grad_(bool(v))

    @property
    def grad(self) -> Optional["Tensor"]:
        g = self._t.grad
        return None if g is None else Tensor(g)

    @grad.setter
    def grad(self, g):
        self._t.grad = None if g is None else _unwrap(g)

    def numel(self) -> int:
        return self._t.numel()

    def data_ptr(self) -> int:
        """Address of the first element; a meta tensor has no storage and raises (reference: Tensor::data_ptr,
        src/tensor/tensor.cpp)."""
        if self._t.device.type == "meta":
            raise RuntimeError("a meta tensor has no data")
        return self._t.data_ptr()

    def element_size(self) -> int:
        """Bytes per stored element (reference: StorageImpl::element_size, include/litetorch/tensor.h)."""
        return self._t.element_size()

    def item(self) -> float:
        return float(self._t.detach().float().reshape(-1)[0].item())

    def to_vector(self) -> List[float]:
        return self._t.detach().float().cpu().reshape(-1).tolist()

    # ---- autograd
    def backward(self, gradient: Optional["Tensor"] = None, create_graph: bool = False):
        g = _unwrap(gradient)
        if g is None and self._t.numel() != 1:
            g = torch.ones_like(self._t)
        self._t.backward(g, create_graph=create_graph, retain_graph=create_graph or None)

    def zero_grad(self):
        self._t.grad = None

    def register_hook(self, fn: Callable[["Tensor"], Optional["Tensor"]]):
        def _hook(g):
            out = fn(Tensor(g))
            return _unwrap(out) if out is not None else None
        return self._t.register_hook(_hook)

    def detach(self) -> "Tensor":
        return Tensor(self._t.detach())

    # ---- movement / layout
    def to(self, device) -> "Tensor":
        out = self._t.to(_as_device(device))
        if self._t.is_leaf and self._t.requires_grad and out is not self._t:
            out = out.detach().requires_grad_(True)
        return Tensor(out, self._dtype_tag)

    def view(self, shape: Sequence[int]) -> "Tensor":
        return Tensor(self._t.view(list(shape)))

    def reshape(self, shape: Sequence[int]) -> "Tensor":
        return Tensor(self._t.reshape(list(shape)))

    def transpose(self, d0: int, d1: int) -> "Tensor":
        return Tensor(self._t.transpose(d0, d1))

    def contiguous(self) -> "Tensor":
        return Tensor(self._t.contiguous())

    def is_contiguous(self) -> bool:
        return self._t.is_contiguous()

    def clone(self) -> "Tensor":
        # a clone is always contiguous in row-major order (reference: Tensor::clone, src/tensor/tensor.cpp)
        return Tensor(self._t.clone(memory_format=torch.contiguous_format), self._dtype_tag)

    def cast(self, target_dtype: DataType) -> "Tensor":
        from .quantization import cast_tensor
        return cast_tensor(self, target_dtype)

    def copy_(self, other: "Tensor") -> "Tensor":
        with torch.no_grad():
            self._t.copy_(_unwrap(other).reshape(self._t.shape))
        return self

    def add_(self, other: "Tensor") -> "Tensor":
        with torch.no_grad():
            self._t.add_(_unwrap(other))
        return self

    def __repr__(self):
        return "lt.Tensor(shape=%s, dtype=%s, device=%s)" % (self.shape, self.dtype.name, self.device)

    # arithmetic sugar (the reference exposes these through lt.Ops only; harmless extras)
    def __add__(self, o): return Tensor(self._t + _unwrap(o))
    def __sub__(self, o): return Tensor(self._t - _unwrap(o))
    def __mul__(self, o): return Tensor(self._t * _unwrap(o))
    def __truediv__(self, o): return Tensor(self._t / _unwrap(o))
    def __neg__(self): return Tensor(-self._t)
    def __radd__(self, o): return Tensor(_unwrap(o) + self._t)
    def __rsub__(self, o): return Tensor(_unwrap(o) - self._t)
    def __rmul__(self, o): return Tensor(_unwrap(o) * self._t)

    def __matmul__(self, o):
        from .ops import Ops                     # the kernel path of Ops.matmul, not a plain torch product
        return Ops.matmul(self, o)


def _gpu_enabled() -> bool:
    """A CUDA device is present and not switched off by the reference's environment variables (LITETORCH_NO_GPU /
    LITETORCH_NO_NATIVE_GPU, src/backend/backend.cpp:115)."""
    if os.environ.get("LITETORCH_NO_GPU") or os.environ.get("LITETORCH_NO_NATIVE_GPU"):
        return False
    return torch.cuda.is_available()


def is_gpu_available() -> bool:
    return _gpu_enabled()


def is_tpu_available() -> bool:
    return False


def auto_device() -> Device:
    """The GPU when there is one and it is not switched off, else the CPU; LITETORCH_DEVICE_INDEX picks the GPU
    (src/cl_backend/cl_backend.cpp:192), otherwise the current CUDA device."""
    if not _gpu_enabled():
        return Device(DeviceType.CPU, 0)
    idx = os.environ.get("LITETORCH_DEVICE_INDEX", "")
    if idx.strip().isdigit() and int(idx) < torch.cuda.device_count():
        return Device(DeviceType.GPU, int(idx))
    return Device(DeviceType.GPU, torch.cuda.current_device())


def get_backend_name() -> str:
    return "CUDA sm_100a (tcgen05/TMA kernels)" if _gpu_enabled() else "CPU"


def checkpoint(fn: Callable, x: Tensor) -> Tensor:
    """Activation checkpointing, function form (src/autograd/checkpoint.cpp:7-64): run `fn` without saving
    activations and recompute them in backward."""
    from torch.utils.checkpoint import checkpoint as _ckpt

    def _f(t):
        return _unwrap(fn(Tensor(t)))
    xt = _unwrap(x)
    if not xt.requires_grad:
        xt = xt.detach().requires_grad_(True)
    return Tensor(_ckpt(_f, xt, use_reentrant=False))


class NoGradGuard:
    def __enter__(self):
        self._g = torch.no_grad()
        self._g.__enter__()
        return self

    def __exit__(self, *a):
        return self._g.__exit__(*a)


def manual_seed(seed: int):
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)
