"""Automatic mixed precision (`lt.amp`): loss scaling and the autocast switch.

`GradScaler` keeps the reference semantics (include/litetorch/amp.h:15-89, src/optim/grad_scaler.cpp:8-79):
scale the loss, check the gradients for inf/nan, skip the step and halve the scale on overflow, otherwise
unscale, step and (every `growth_interval` clean steps) double the scale, never below 1.0.  On CUDA the
check is one fused reduction kernel per gradient (sum of squares + non-finite count) instead of the
reference's `Ops::max(Ops::abs(g))` chain.
`AutocastGuard(enabled, dtype)` is consumed by `Ops.matmul` and `Ops.flash_attention`; it also works as a
context manager, which the reference's README shows but its binding lacks.
"""
from __future__ import annotations

import threading

import torch

from .core import DataType, Tensor, _TO_TORCH, _unwrap

_state = threading.local()


class AutocastGuard:
    def __init__(self, enabled: bool = True, dtype: DataType = DataType.BF16):
        self._prev = (getattr(_state, "enabled", False), getattr(_state, "dtype", DataType.BF16))
        _state.enabled, _state.dtype = bool(enabled), dtype
        self._active = True

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()
        return False

    def close(self):
        if self._active:
            _state.enabled, _state.dtype = self._prev
            self._active = False

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @staticmethod
    def is_enabled() -> bool:
        return getattr(_state, "enabled", False)

    @staticmethod
    def get_dtype() -> DataType:
        return getattr(_state, "dtype", DataType.BF16)

    @staticmethod
    def torch_dtype():
        return _TO_TORCH[AutocastGuard.get_dtype()]


def _has_overflow(params) -> bool:
    bad = False
    cuda_stats = None
    for p in params:
        g = _unwrap(p).grad
        if g is None:
            continue
        if g.is_cuda and g.dtype in (torch.float32, torch.bfloat16) and g.is_contiguous():
            from .ops import kernels as K
            if cuda_stats is None:
                cuda_stats = torch.zeros(2, device=g.device)
            K.sumsq(g, cuda_stats)
        else:
            bad = bad or not bool(torch.isfinite(g).all())
    if cuda_stats is not None:
        s = cuda_stats.tolist()
        bad = bad or s[1] != 0.0 or s[0] != s[0] or s[0] == float("inf")
    return bad


class GradScaler:
    def __init__(self, init_scale: float = 65536.0, growth_factor: float = 2.0, backoff_factor: float = 0.5,
                 growth_interval: int = 2000):
        self._scale = float(init_scale)
        self.growth_factor, self.backoff_factor, self.growth_interval = growth_factor, backoff_factor, growth_interval
        self._good_steps = 0
        self._found_inf = False

    # reference names: scale / step / update / get_scale   (optim.GradScaler: scale_loss / step / update / .scale)
    def scale(self, loss: Tensor) -> Tensor:
        return Tensor(_unwrap(loss) * self._scale)

    scale_loss = scale

    def get_scale(self) -> float:
        return self._scale

    def step(self, optimizer) -> bool:
        params = optimizer.params
        grads = [_unwrap(p).grad for p in params if _unwrap(p).grad is not None]
        inv = 1.0 / self._scale
        if grads and all(g.is_cuda and g.is_contiguous() and g.dtype in (torch.float32, torch.bfloat16) for g in grads):
            # one pass per gradient: unscale and look for inf / nan together; a single flag read at the end
            from .ops import kernels as K
            flag = torch.zeros(1, dtype=torch.int32, device=grads[0].device)
            with torch.no_grad():
                for g in grads:
                    K.unscale_check_(g, inv, flag)
            self._found_inf = bool(flag.item())
            if self._found_inf:
                return False     # the gradients are discarded by the caller's zero_grad; the scale backs off in update()
            optimizer.step()
            return True
        self._found_inf = _has_overflow(params)
        if self._found_inf:
            return False
        with torch.no_grad():
            for g in grads:
                g.mul_(inv)
        optimizer.step()
        return True

    def update(self) -> None:
        if self._found_inf:
            self._scale = max(self._scale * self.backoff_factor, 1.0)
            self._good_steps = 0
        else:
            self._good_steps += 1
            if self._good_steps >= self.growth_interval:
                self._scale *= self.growth_factor
                self._good_steps = 0
        self._found_inf = False
