"""`lt.Ops`: the functional API of the reference (include/litetorch/ops.h:11-110, bound at
src/bindings/python_bindings.cpp:258-314) over `lt.Tensor`.

Hot ops (matmul, layer/RMS norm, GELU, SwiGLU, RoPE, flash attention, cross-entropy, embedding) reach the
sm_100a kernels for CUDA bf16 tensors through `functional.py`; the long tail runs on PyTorch's native ops.
Additions the reference's README claims but its sources lack: `rms_norm`, `silu`, `swiglu`, and the
`is_causal` argument of `flash_attention`.
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

from ..core import DataType, Tensor, _unwrap
from . import functional as Fn


def _w(t: torch.Tensor) -> Tensor:
    return Tensor(t)


class Ops:
    # ------------------------------------------------------------------ elementwise (NumPy broadcasting)
    @staticmethod
    def add(a, b): return _w(_unwrap(a) + _unwrap(b))
    @staticmethod
    def sub(a, b): return _w(_unwrap(a) - _unwrap(b))
    @staticmethod
    def mul(a, b): return _w(_unwrap(a) * _unwrap(b))
    @staticmethod
    def div(a, b): return _w(_unwrap(a) / _unwrap(b))
    @staticmethod
    def pow(a, exponent: float): return _w(torch.pow(_unwrap(a), exponent))
    @staticmethod
    def sqrt(a): return _w(torch.sqrt(_unwrap(a)))
    @staticmethod
    def exp(a): return _w(torch.exp(_unwrap(a)))
    @staticmethod
    def log(a): return _w(torch.log(_unwrap(a)))
    @staticmethod
    def abs(a): return _w(torch.abs(_unwrap(a)))
    @staticmethod
    def neg(a): return _w(-_unwrap(a))
    @staticmethod
    def clamp(a, min_val: float, max_val: float): return _w(torch.clamp(_unwrap(a), min_val, max_val))
    @staticmethod
    def sin(a): return _w(torch.sin(_unwrap(a)))
    @staticmethod
    def cos(a): return _w(torch.cos(_unwrap(a)))

    # ------------------------------------------------------------------ reductions (full reduce to shape [1])
    @staticmethod
    def sum(a):
        t = _unwrap(a)
        if t.is_cuda and not t.requires_grad and t.dtype in (torch.float32, torch.bfloat16) and t.numel() > 0:
            from . import kernels as K
            return _w(K.reduce_all(t, "sum").to(t.dtype))
        return _w(t.sum().reshape(1))
    @staticmethod
    def mean(a): return _w(_unwrap(a).mean().reshape(1))
    @staticmethod
    def max(a):
        t = _unwrap(a)
        if t.is_cuda and not t.requires_grad and t.dtype in (torch.float32, torch.bfloat16) and t.numel() > 0:
            from . import kernels as K
            return _w(K.reduce_all(t, "max").to(t.dtype))
        return _w(t.max().reshape(1))

    # ------------------------------------------------------------------ shape
    @staticmethod
    def cat(tensors: Sequence[Tensor], dim: int = 0): return _w(torch.cat([_unwrap(t) for t in tensors], dim))
    @staticmethod
    def squeeze(a, dim: int = -1): return _w(_unwrap(a).squeeze(dim))
    @staticmethod
    def unsqueeze(a, dim: int): return _w(_unwrap(a).unsqueeze(dim))
    @staticmethod
    def cast(a, target_dtype: DataType): return a.cast(target_dtype)

    # ------------------------------------------------------------------ GEMM
    @staticmethod
    def matmul(a, b):
        from ..amp import AutocastGuard
        ta, tb = _unwrap(a), _unwrap(b)
        if AutocastGuard.is_enabled() and ta.is_floating_point():
            dt = AutocastGuard.torch_dtype()
            ta, tb = ta.to(dt), tb.to(dt)
        return _w(Fn.matmul(ta, tb))

    @staticmethod
    def bmm(a, b): return _w(Fn.bmm(_unwrap(a), _unwrap(b)))

    @staticmethod
    def scaled_matmul(a, b, a_scale: float, b_scale: float, bias=None, out_dtype: DataType = DataType.FP32):
        """Low-precision operands with per-tensor scales: (a @ b) * a_scale * b_scale + bias (src/ops/scaled_matmul.cpp:8-43)."""
        from ..quantization import to_float
        at, bt = _unwrap(a), _unwrap(b)
        if (at.is_cuda and at.dtype == torch.float8_e4m3fn and bt.dtype == torch.float8_e4m3fn and at.dim() == 2 and bt.dim() == 2
                and at.shape[1] % 16 == 0 and at.numel() > 0 and bt.numel() > 0):
            # e4m3 codes on the tensor cores (tcgen05 kind::f8f6f4, fp32 accumulation over the whole K extent); b is [K, N]:
            # its codes are laid out K-major first
            from . import kernels as K
            y = K.gemm_e4m3(at.contiguous(), None, bt.t().contiguous(), None, out_dtype=torch.float32, alpha=float(a_scale * b_scale))
        else:
            y = torch.matmul(to_float(a), to_float(b)) * (a_scale * b_scale)
        if bias is not None:
            y = y + _unwrap(bias).float()
        return _w(y).cast(out_dtype)

    @staticmethod
    def w8a8_matmul(x, w, x_scale: float, w_scale: float):
        """int8 x int8 with int32 accumulation and per-tensor scales: x [M, K], w [N, K] (one row per output feature, the
        layout of a Linear weight), result [M, N] = (q(x) @ q(w)^T) * x_scale * w_scale (src/ops/w8a8_ops.cpp:28-107)."""
        xt, wt = _unwrap(x), _unwrap(w)
        if xt.dim() != 2 or wt.dim() != 2:
            raise ValueError("w8a8_matmul expects 2-D inputs")
        if wt.shape[1] != xt.shape[1]:
            raise ValueError("inner dimensions differ in w8a8_matmul: x %s, w %s" % (list(xt.shape), list(wt.shape)))
        if (xt.is_cuda and xt.dtype in (torch.float32, torch.bfloat16) and wt.dtype == xt.dtype
                and xt.shape[1] % 16 == 0 and xt.numel() > 0 and wt.numel() > 0):
            # quantiser kernels + the tcgen05 int8 GEMM (exact int32 sums); both operands are K-major as they stand
            from . import kernels as K
            xq = K.quant_int8_tensor(xt.contiguous(), x_scale)
            wq = K.quant_int8_tensor(wt.contiguous(), w_scale)
            return _w(K.gemm_i8(xq, wq, alpha=x_scale * w_scale))
        xq = torch.clamp(torch.round(xt.float() / x_scale), -127, 127)
        wq = torch.clamp(torch.round(wt.float() / w_scale), -127, 127)
        return _w(torch.matmul(xq, wq.t()) * (x_scale * w_scale))

    # ------------------------------------------------------------------ activations
    @staticmethod
    def relu(a): return _w(torch.relu(_unwrap(a)))
    @staticmethod
    def leaky_relu(a, negative_slope: float = 0.01): return _w(F.leaky_relu(_unwrap(a), negative_slope))
    @staticmethod
    def sigmoid(a): return _w(torch.sigmoid(_unwrap(a)))
    @staticmethod
    def tanh(a): return _w(torch.tanh(_unwrap(a)))
    @staticmethod
    def silu(a): return _w(F.silu(_unwrap(a)))
    @staticmethod
    def softmax(a, dim: int = -1): return _w(Fn.softmax(_unwrap(a), dim))
    @staticmethod
    def gelu(a): return _w(Fn.gelu(_unwrap(a)))
    @staticmethod
    def swiglu(gate_up): return _w(Fn.swiglu(_unwrap(gate_up)))

    # ------------------------------------------------------------------ normalisation
    @staticmethod
    def layer_norm(input, normalized_shape, weight=None, bias=None, eps: float = 1e-5):
        t = _unwrap(input)
        D = t.shape[-1]
        if len(list(normalized_shape)) == 1 and weight is not None and bias is not None:
            return _w(Fn.layer_norm(t, _unwrap(weight), _unwrap(bias), eps))
        return _w(F.layer_norm(t, list(normalized_shape), _unwrap(weight), _unwrap(bias), eps))

    @staticmethod
    def fused_add_layernorm(input, residual, normalized_shape, weight=None, bias=None, eps: float = 1e-5):
        t, r = _unwrap(input), _unwrap(residual)
        if len(list(normalized_shape)) == 1 and weight is not None and bias is not None:
            return _w(Fn.layer_norm(t, _unwrap(weight), _unwrap(bias), eps, residual=r))
        return _w(F.layer_norm(t + r, list(normalized_shape), _unwrap(weight), _unwrap(bias), eps))

    @staticmethod
    def rms_norm(x, weight, eps: float = 1e-5, residual=None):
        return _w(Fn.rms_norm(_unwrap(x), _unwrap(weight), eps, _unwrap(residual)))

    @staticmethod
    def batch_norm2d(input, running_mean, running_var, weight, bias, training: bool, momentum: float = 0.1, eps: float = 1e-5):
        t = _unwrap(input)
        if training and t.dim() >= 2 and t.numel() == t.shape[1]:
            # one value per channel: the batch variance is 0 and its unbiased factor M / (M - 1) is taken as 1
            # (reference: src/ops/normalization.cpp:650), where torch refuses the call
            rm, rv = _unwrap(running_mean), _unwrap(running_var)
            with torch.no_grad():
                rm.mul_(1 - momentum).add_(t.detach().reshape(-1).to(rm.dtype), alpha=momentum)
                rv.mul_(1 - momentum)
            shape = [1, -1] + [1] * (t.dim() - 2)
            out = (t - t.detach()) * torch.rsqrt(torch.zeros((), dtype=t.dtype, device=t.device) + eps)
            if weight is not None:
                out = out * _unwrap(weight).view(shape)
            if bias is not None:
                out = out + _unwrap(bias).view(shape)
            return _w(out)
        return _w(F.batch_norm(t, _unwrap(running_mean), _unwrap(running_var), _unwrap(weight), _unwrap(bias),
                               training, momentum, eps))

    # ------------------------------------------------------------------ vision
    @staticmethod
    def conv2d(input, weight, bias=None, stride: int = 1, padding: int = 0):
        return _w(F.conv2d(_unwrap(input), _unwrap(weight), _unwrap(bias), stride, padding))
    @staticmethod
    def conv3d(input, weight, bias=None, stride: int = 1, padding: int = 0):
        return _w(F.conv3d(_unwrap(input), _unwrap(weight), _unwrap(bias), stride, padding))
    @staticmethod
    def max_pool2d(input, kernel_size: int, stride: int = -1, padding: int = 0):
        return _w(F.max_pool2d(_unwrap(input), kernel_size, kernel_size if stride <= 0 else stride, padding))
    @staticmethod
    def max_pool3d(input, kernel_size: int, stride: int = -1, padding: int = 0):
        return _w(F.max_pool3d(_unwrap(input), kernel_size, kernel_size if stride <= 0 else stride, padding))
    @staticmethod
    def adaptive_avg_pool2d(input, output_height: int, output_width: int):
        return _w(F.adaptive_avg_pool2d(_unwrap(input), (output_height, output_width)))

    # ------------------------------------------------------------------ losses
    @staticmethod
    def mse_loss(x, target): return _w(F.mse_loss(_unwrap(x), _unwrap(target)).reshape(1))
    @staticmethod
    def l1_loss(x, target): return _w(F.l1_loss(_unwrap(x), _unwrap(target)).reshape(1))
    @staticmethod
    def bce_loss(x, target):
        p = torch.clamp(_unwrap(x), 1e-7, 1 - 1e-7)
        return _w(F.binary_cross_entropy(p, _unwrap(target)).reshape(1))
    @staticmethod
    def cross_entropy_loss(logits, target):
        """Mean CE of logits [N, C] against class indices [N] stored as floats or integers.  A floating-point target of the
        logits' own shape is read as class probabilities per row (the reference's AMP guide passes such a target,
        docs-en/7.optimizers_and_amp.md, though its own op insists on a 1-D target, src/ops/loss.cpp:373-375)."""
        lt_, tt = _unwrap(logits), _unwrap(target)
        if tt.dim() == 2 and tt.shape == lt_.shape and tt.is_floating_point():
            return _w(F.cross_entropy(lt_.float(), tt.float()).reshape(1))
        return _w(Fn.cross_entropy(lt_, tt).reshape(1))

    @staticmethod
    def fused_linear_cross_entropy(x, weight, target, bias=None, chunk_rows: int = 4096):
        """CE(x @ weight^T + bias, target) without keeping the full logits: rows are processed in chunks and each
        chunk's logits are recomputed in backward (src/ops/fused_loss.cpp:12-195)."""
        from torch.utils.checkpoint import checkpoint as ckpt
        xt, wt, tt = _unwrap(x), _unwrap(weight), _unwrap(target).to(torch.int64)
        bt = _unwrap(bias)
        if bt is None:
            # CUDA bf16: chunks on the tcgen05 GEMM and the cross-entropy kernels, gradients formed in the forward
            # pass, nothing recomputed and no [N, V] tensor at any time
            fused = Fn.fused_linear_cross_entropy(xt, wt, tt, chunk_rows)
            if fused is not None:
                return _w(fused.reshape(1))
        N = xt.shape[0]
        total = xt.new_zeros((), dtype=torch.float32)

        def piece(xc, tc):
            return F.cross_entropy(Fn.linear(xc, wt, bt).float(), tc, reduction="sum")
        for s in range(0, N, chunk_rows):
            xc, tc = xt[s:s + chunk_rows], tt[s:s + chunk_rows]
            total = total + (ckpt(piece, xc, tc, use_reentrant=False) if torch.is_grad_enabled() else piece(xc, tc))
        return _w((total / N).reshape(1))

    @staticmethod
    def clip_grad_norm_(params: Sequence[Tensor], max_norm: float, norm_type: float = 2.0) -> float:
        ts = [_unwrap(p) for p in params if _unwrap(p).grad is not None]
        if not ts:
            return 0.0
        return float(torch.nn.utils.clip_grad_norm_(ts, max_norm, norm_type))

    # ------------------------------------------------------------------ transformer ops
    @staticmethod
    def rope(x, cos, sin):
        """Interleaved-pair rotary embedding of x [B, H, T, D] with cos/sin [T, D/2]."""
        return _w(Fn.rope(_unwrap(x), _unwrap(cos), _unwrap(sin)))

    @staticmethod
    def flash_attention(q, k, v, is_causal: bool = False, scale: Optional[float] = None):
        """softmax(Q K^T * scale [+ causal mask]) V for [B, H, T, D] tensors; K/V may have fewer heads (GQA)."""
        from ..amp import AutocastGuard
        tq, tk, tv = _unwrap(q), _unwrap(k), _unwrap(v)
        if AutocastGuard.is_enabled():
            dt = AutocastGuard.torch_dtype()
            tq, tk, tv = tq.to(dt), tk.to(dt), tv.to(dt)
        return _w(Fn.flash_attention(tq, tk, tv, is_causal, scale))

    @staticmethod
    def paged_attention(q, k_cache, v_cache, block_tables, context_lens, block_size: int):
        from ..serving import paged_attention
        qt, kt, vt = _unwrap(q), _unwrap(k_cache), _unwrap(v_cache)
        if kt.dim() == 3:        # [num_blocks, block_size, head_dim]: one KV head (the layout the reference's serving guide uses)
            kt, vt = kt.unsqueeze(1), vt.unsqueeze(1)
        return _w(paged_attention(qt, kt, vt, _unwrap(block_tables), _unwrap(context_lens), block_size))

    @staticmethod
    def flash_decoding(q, k, v, num_splits: int = 4):
        """Split-K decode attention for Tq == 1: per-split (max, sum, partial output) merged at the end
        (src/ops/flash_decoding.cpp:13-115)."""
        qt, kt, vt = _unwrap(q), _unwrap(k), _unwrap(v)
        if (qt.is_cuda and qt.dtype == torch.bfloat16 and qt.dim() == 4 and qt.shape[2] == 1 and qt.shape[-1] in (64, 128)
                and kt.dtype == torch.bfloat16 and kt.is_contiguous() and vt.is_contiguous()):
            # q [B, H, 1, D], k / v [B, Hkv, T, D]: a contiguous KV tensor is a paged cache with one block of T keys per
            # sequence, so the split-K paged kernel (a warp per sequence, head and split; a merge kernel) serves it.
            from . import kernels as K
            B, H, _, D = qt.shape
            T = kt.shape[2]
            bt = torch.arange(B, dtype=torch.int32, device=qt.device).view(B, 1)
            cl = torch.full((B,), T, dtype=torch.int32, device=qt.device)
            o = K.paged_decode(qt.reshape(B, H, D).contiguous(), kt, vt, bt, cl, T, max(1, min(int(num_splits), 32)), D ** -0.5)
            return _w(o.view(B, H, 1, D))
        tq, tk, tv = qt.float(), kt.float(), vt.float()
        G = tq.shape[1] // tk.shape[1]
        if G > 1:
            tk, tv = tk.repeat_interleave(G, 1), tv.repeat_interleave(G, 1)
        scale = tq.shape[-1] ** -0.5
        T = tk.shape[2]
        step = (T + num_splits - 1) // num_splits
        m = None
        for s in range(0, T, step):
            sc = torch.matmul(tq, tk[:, :, s:s + step].transpose(-1, -2)) * scale
            ms = sc.amax(-1, keepdim=True)
            p = torch.exp(sc - ms)
            ls = p.sum(-1, keepdim=True)
            os_ = torch.matmul(p, tv[:, :, s:s + step])
            if m is None:
                m, l, o = ms, ls, os_
            else:
                nm = torch.maximum(m, ms)
                a, b = torch.exp(m - nm), torch.exp(ms - nm)
                l = l * a + ls * b
                o = o * a + os_ * b
                m = nm
        return _w((o / l).to(_unwrap(q).dtype))

    @staticmethod
    def ring_attention(q, k, v, pg=None, causal: bool = False):
        from ..parallel.cp import ring_attention
        return _w(ring_attention(_unwrap(q), _unwrap(k), _unwrap(v), pg, causal=causal))

    @staticmethod
    def moe_gate(x, gate_weight, top_k: int) -> Tuple[Tensor, Tensor]:
        """logits = x @ Wg^T -> softmax over experts (fp32) -> top-k -> renormalise.  Returns (probs [N,k], indices [N,k]
        as floats), as src/ops/moe_ops.cpp:11-106."""
        xt, wt = _unwrap(x), _unwrap(gate_weight)
        logits = F.linear(xt.float(), wt.float())
        # the warp-per-token router kernel on CUDA (fp32 softmax, top-k, renormalisation; differentiable), torch elsewhere
        top_p, top_i, _ = Fn.moe_router(logits.reshape(-1, logits.shape[-1]), top_k, True)
        lead = tuple(logits.shape[:-1])
        return _w(top_p.reshape(*lead, top_k)), _w(top_i.reshape(*lead, top_k).to(torch.float32))

    @staticmethod
    def fake_quantize(input, scale: float, zero_point: float = 0.0, bits: int = 8):
        from ..quantization import fake_quantize
        return _w(fake_quantize(_unwrap(input), scale, zero_point, bits))

    @staticmethod
    def checkpoint(module, input):
        """Activation checkpointing, module form (src/ops/checkpoint.cpp:8-96)."""
        from torch.utils.checkpoint import checkpoint as ckpt
        xt = _unwrap(input)
        if not xt.requires_grad:
            xt = xt.detach().requires_grad_(True)
        return _w(ckpt(lambda t: _unwrap(module.forward(Tensor(t))), xt, use_reentrant=False))


__all__ = ["Ops"]
