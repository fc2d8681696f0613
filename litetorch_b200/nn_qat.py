"""QATLinear: Linear with fake-quantised weights and activations while training
(include/litetorch/quantization.h:93-141)."""
from __future__ import annotations

import torch

from .core import Tensor, _as_device, _unwrap


class QATLinear:
    def __init__(self, linear, w_scale: float = 0.01, w_zp: float = 0.0, a_scale: float = 0.01, a_zp: float = 0.0, b: int = 8,
                 bits: int = None):
        """`b` is the bit width under the reference's keyword (src/bindings/python_bindings.cpp:710-711); `bits` is accepted too."""
        self.weight, self.bias = linear.weight, linear.bias
        self.weight_scale, self.weight_zero_point = w_scale, w_zp
        self.act_scale, self.act_zero_point = a_scale, a_zp
        self.bits = int(b if bits is None else bits)
        self.qat_enabled = True
        self.training = True

    def forward(self, x: Tensor) -> Tensor:
        from .quantization import fake_quantize
        w, xt = _unwrap(self.weight), _unwrap(x)
        if self.qat_enabled and self.training:
            w = fake_quantize(w, self.weight_scale, self.weight_zero_point, self.bits)
            xt = fake_quantize(xt, self.act_scale, self.act_zero_point, self.bits)
        return Tensor(torch.nn.functional.linear(xt, w, _unwrap(self.bias) if self.bias is not None else None))

    __call__ = forward

    def parameters(self):
        return [self.weight] + ([self.bias] if self.bias is not None else [])

    def train(self, mode=True):
        self.training = mode
        return self

    def eval(self):
        return self.train(False)

    def to(self, device):
        d = _as_device(device)
        self.weight = Tensor(_unwrap(self.weight).detach().to(d).requires_grad_(True))
        if self.bias is not None:
            self.bias = Tensor(_unwrap(self.bias).detach().to(d).requires_grad_(True))
        return self
