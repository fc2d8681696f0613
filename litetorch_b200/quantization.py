"""Low-precision codecs and quantisation helpers (`lt.quantization`).

* `cast_tensor` implements `Tensor.cast` for every pair of the 11 data types.  fp16/bf16/fp8 use the
  hardware conversions of PyTorch; the 4-bit formats (NF4, FP4 E2M1, INT4) are stored one code per byte as
  in the reference (src/tensor/tensor_core.cpp:39-153) and dequantise through their code books.
* `quantize_linear` (per-output-row absmax int8), `Calibrator` (running min/max -> symmetric or asymmetric
  parameters) and `QATLinear` (fake-quantised weights and activations, straight-through gradient) follow
  include/litetorch/quantization.h:15-141.
* `quantize_fp8_1x128` / `quantize_fp8_128x128`: e4m3 with one fp32 scale per 1x128 activation block or
  128x128 weight block, the scaling layout of the fp8 training configuration.
"""
from __future__ import annotations

from typing import Dict, Tuple

import torch

from .core import DataType, Tensor, _TO_TORCH, _unwrap

NF4_CODEBOOK = torch.tensor([-1.0, -0.6961928009986877, -0.5250730514526367, -0.39491748809814453, -0.28444138169288635,
                             -0.18477343022823334, -0.09105003625154495, 0.0, 0.07958029955625534, 0.16093020141124725,
                             0.24611230194568634, 0.33791524171829224, 0.44070982933044434, 0.5626170039176941,
                             0.7229568362236023, 1.0])
FP4_CODEBOOK = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0])


def _nearest_code(x: torch.Tensor, book: torch.Tensor) -> torch.Tensor:
    book = book.to(x.device)
    return (x.unsqueeze(-1) - book).abs().argmin(-1).to(torch.uint8)


def to_float(t) -> torch.Tensor:
    """fp32 view of any lt.Tensor / torch tensor, decoding the byte-per-code 4-bit formats."""
    if isinstance(t, Tensor) and t._dtype_tag in (DataType.NF4, DataType.FP4_E2M1, DataType.INT4):
        raw = t._t
        if t._dtype_tag == DataType.NF4:
            return NF4_CODEBOOK.to(raw.device)[raw.long()]
        if t._dtype_tag == DataType.FP4_E2M1:
            return FP4_CODEBOOK.to(raw.device)[raw.long()]
        return raw.to(torch.int8).float()
    return _unwrap(t).float()


def cast_tensor(t: Tensor, dtype: DataType) -> Tensor:
    x = to_float(t)
    if dtype == DataType.NF4:
        return Tensor(_nearest_code(torch.clamp(x, -1.0, 1.0), NF4_CODEBOOK), DataType.NF4)
    if dtype == DataType.FP4_E2M1:
        return Tensor(_nearest_code(torch.clamp(x, -6.0, 6.0), FP4_CODEBOOK), DataType.FP4_E2M1)
    # integer targets clamp and then drop the fraction, as a C cast does (src/tensor/tensor_core.cpp:1102-1117: 1.5 -> 1, -2.5 -> -2)
    if dtype == DataType.INT4:
        return Tensor(torch.trunc(torch.clamp(x, -8, 7)).to(torch.int8), DataType.INT4)
    if dtype in (DataType.INT8, DataType.INT16):
        lim = 127 if dtype == DataType.INT8 else 32767
        return Tensor(torch.trunc(torch.clamp(x, -lim - 1, lim)).to(_TO_TORCH[dtype]))
    if dtype == DataType.FP8_E4M3:
        return Tensor(torch.clamp(x, -448.0, 448.0).to(torch.float8_e4m3fn))
    if dtype == DataType.FP8_E5M2:
        return Tensor(torch.clamp(x, -57344.0, 57344.0).to(torch.float8_e5m2))
    src = _unwrap(t)
    if t._dtype_tag is None and src.is_floating_point() and src.requires_grad:
        return Tensor(src.to(_TO_TORCH[dtype]))  # stays on the autograd tape (CastNode in the reference)
    return Tensor(x.to(_TO_TORCH[dtype]))


class _FakeQuant(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, scale, zero_point, bits):
        qmax = 2.0 ** (bits - 1) - 1
        q = torch.clamp(torch.round(x / scale + zero_point), -qmax - 1, qmax)
        return (q - zero_point) * scale

    @staticmethod
    def backward(ctx, g):  # straight-through estimator
        return g, None, None, None


def fake_quantize(x: torch.Tensor, scale: float, zero_point: float = 0.0, bits: int = 8) -> torch.Tensor:
    return _FakeQuant.apply(x, float(scale), float(zero_point), int(bits))


def quantize_linear(layer) -> None:
    """Replace `layer.weight` by int8 codes with one scale per output row (dequantised on the fly in forward)."""
    Wt = _unwrap(layer.weight).detach()
    if Wt.is_cuda and Wt.dim() == 2 and Wt.dtype in (torch.float32, torch.bfloat16):
        from .ops import kernels as K                  # warp-per-row absmax + rounding kernel
        q, scales = K.quant_int8_rows(Wt)
    else:
        W = Wt.float()
        amax = W.abs().amax(1)
        scales = torch.where(amax > 0, amax / 127.0, torch.ones_like(amax))
        q = torch.round(W / scales[:, None]).to(torch.int8)
    layer.weight = Tensor(q)
    layer.scales = Tensor(scales)


class Calibrator:
    def __init__(self):
        self.min_vals: Dict[str, float] = {}
        self.max_vals: Dict[str, float] = {}

    def collect(self, name: str, tensor) -> None:
        t = _unwrap(tensor).detach().float()
        lo, hi = (float(t.min()), float(t.max())) if t.numel() else (0.0, 0.0)
        if name not in self.min_vals:
            self.min_vals[name], self.max_vals[name] = lo, hi
        else:
            self.min_vals[name] = min(self.min_vals[name], lo)
            self.max_vals[name] = max(self.max_vals[name], hi)

    def get_asymmetric_params(self, name: str, bits: int = 8) -> Tuple[float, float]:
        if name not in self.min_vals:
            return 1.0, 0.0
        lo, hi = self.min_vals[name], self.max_vals[name]
        bound = 2.0 ** (bits - 1) - 1.0
        qmin, qmax = -bound, bound
        scale = (hi - lo) / (qmax - qmin)
        if scale == 0.0:
            scale = 1.0
        zp = float(round(-lo / scale + qmin))
        return scale, min(max(zp, qmin), qmax)

    def get_scale(self, name: str, bits: int = 8) -> float:
        if name not in self.max_vals:
            return 1.0
        m = max(abs(self.min_vals[name]), abs(self.max_vals[name]))
        bound = 2.0 ** (bits - 1) - 1.0
        return m / bound if m > 0 else 1.0


def quantize_fp8_1x128(x: torch.Tensor):
    """Activations: e4m3 codes and one fp32 scale per 1 x 128 block of the last dimension."""
    M, Kd = x.shape
    assert Kd % 128 == 0
    xb = x.float().view(M, Kd // 128, 128)
    amax = xb.abs().amax(-1).clamp_min(1e-12)
    scale = amax / 448.0
    q = (xb / scale[..., None]).clamp(-448, 448).to(torch.float8_e4m3fn).view(M, Kd)
    return q, scale


def quantize_fp8_128x128(w: torch.Tensor):
    """Weights: e4m3 codes and one fp32 scale per 128 x 128 block."""
    N, Kd = w.shape
    if w.is_cuda and w.dtype == torch.bfloat16 and Kd % 128 == 0:
        from .ops import kernels as K
        return K.quant_fp8_128x128(w.contiguous())
    assert N % 128 == 0 and Kd % 128 == 0
    wb = w.float().view(N // 128, 128, Kd // 128, 128)
    amax = wb.abs().amax((1, 3)).clamp_min(1e-12)
    scale = amax / 448.0
    q = (wb / scale[:, None, :, None]).clamp(-448, 448).to(torch.float8_e4m3fn).view(N, Kd)
    return q, scale


def fp8_block_linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """y = x @ w^T with both operands rounded to block-scaled e4m3 (1x128 / 128x128) and fp32 accumulation.
    On a GPU the product runs on the tcgen05 fp8 kernel (two-level accumulation, fp32 scales); on the host the same
    arithmetic is carried out on dequantised values."""
    if x.is_cuda and x.dtype == torch.bfloat16:
        from .ops import kernels as K
        xq, xst = K.quant_fp8_1x128(x.contiguous())
        wq, ws = quantize_fp8_128x128(w)
        return K.gemm_fp8_block(xq, xst, wq, ws.contiguous())
    xq, xs = quantize_fp8_1x128(x)
    wq, ws = quantize_fp8_128x128(w)
    xd = (xq.float().view(x.shape[0], -1, 128) * xs[..., None]).view_as(x)
    wd = (wq.float().view(w.shape[0] // 128, 128, -1, 128) * ws[:, None, :, None]).view_as(w)
    return (xd @ wd.t()).to(x.dtype)


from .nn_qat import QATLinear  # noqa: E402  (needs nn.Module; defined separately to avoid an import cycle)
