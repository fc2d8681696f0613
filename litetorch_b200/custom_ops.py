"""Custom operator registry (`lt.custom_ops.Registry`): name -> forward / backward callables, differentiable.

Mirrors include/litetorch/custom_ops.h:16-45 (cpu_forward, gpu_forward, backward closures + CustomOpNode): an op is
registered once and called by name; its backward receives the saved inputs, the output and the incoming gradient and
returns one gradient per input.
"""
from __future__ import annotations

from typing import Callable, Dict, Optional, Sequence

import torch

from .core import Tensor, _unwrap


class _Entry:
    def __init__(self, cpu_forward, gpu_forward, backward):
        self.cpu_forward, self.gpu_forward, self.backward = cpu_forward, gpu_forward, backward


class _Apply(torch.autograd.Function):
    @staticmethod
    def forward(ctx, entry, *inputs):
        fn = entry.gpu_forward if (inputs and inputs[0].is_cuda and entry.gpu_forward is not None) else entry.cpu_forward
        out = _unwrap(fn(*[Tensor(t) for t in inputs]))
        ctx.entry = entry
        ctx.save_for_backward(*inputs, out)
        return out

    @staticmethod
    def backward(ctx, g):
        *inputs, out = ctx.saved_tensors
        if ctx.entry.backward is None:
            raise RuntimeError("custom op has no backward")
        grads = ctx.entry.backward([Tensor(t) for t in inputs], Tensor(out), Tensor(g))
        if not isinstance(grads, (list, tuple)):
            grads = [grads]
        return (None,) + tuple(None if x is None else _unwrap(x) for x in grads)


class Registry:
    _ops: Dict[str, _Entry] = {}

    @classmethod
    def register(cls, name: str, cpu_forward: Callable, backward: Optional[Callable] = None, gpu_forward: Optional[Callable] = None):
        cls._ops[name] = _Entry(cpu_forward, gpu_forward, backward)

    # the C++ spelling of the reference: custom_ops::Registry::get().register_op(name, cpu_forward, gpu_forward, backward)
    @classmethod
    def get(cls) -> "type":
        return cls

    @classmethod
    def register_op(cls, name: str, cpu_forward: Callable, gpu_forward: Optional[Callable] = None, backward: Optional[Callable] = None):
        """The reference's calling conventions (include/litetorch/custom_ops.h): forward(list of tensors) -> tensor,
        backward(grad_output, list of inputs, output) -> list of gradients."""
        def fwd(f):
            return None if f is None else (lambda *ts: f(list(ts)))
        bwd = None if backward is None else (lambda inputs, out, g: backward(g, list(inputs), out))
        cls.register(name, fwd(cpu_forward), bwd, fwd(gpu_forward))

    @classmethod
    def has(cls, name: str) -> bool:
        return name in cls._ops

    @classmethod
    def call(cls, name: str, inputs: Sequence[Tensor]) -> Tensor:
        if name not in cls._ops:
            raise KeyError("custom op %r is not registered" % name)
        return Tensor(_Apply.apply(cls._ops[name], *[_unwrap(t) for t in inputs]))

    @classmethod
    def unregister(cls, name: str):
        cls._ops.pop(name, None)
