"""Autograd-aware functional ops on torch tensors.

CUDA bf16 inputs run on the sm_100a kernels (tcgen05 GEMM, FlashAttention, fused norms, RoPE, SwiGLU,
cross-entropy) through hand-written `torch.autograd.Function`s; anything else (CPU tensors, fp32/fp64 on
the GPU, shapes the kernels do not cover) runs the same math in stock PyTorch, which is also the oracle
the GPU tests compare against.  A CUDA bf16 call never falls back silently when the native library is
missing: loading it raises.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn.functional as F

from . import kernels as K


def _native(*ts) -> bool:
    for t in ts:
        if t is None:
            continue
        if not (t.is_cuda and t.dtype == torch.bfloat16):
            return False
    return True


def _2d(x):
    return x.reshape(-1, x.shape[-1])


# ---------------------------------------------------------------------------------------------- linear / matmul
class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, b, act):
        x2 = _2d(x).contiguous()
        wc = w.contiguous()
        pre = None
        if act == 1 and (x.requires_grad or w.requires_grad):
            pre = K.gemm(x2, wc, bias=b)
            y = K.gelu_fwd(pre)
        else:
            y = K.gemm(x2, wc, bias=b, act=act)
        ctx.save_for_backward(x2, wc, pre)
        ctx.has_bias = b is not None
        ctx.act = act
        ctx.xshape = x.shape
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w, pre = ctx.saved_tensors
        dy2 = _2d(dy).contiguous()
        if ctx.act == 1:
            dy2 = K.gelu_bwd(pre, dy2)
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = K.gemm(dy2, w, b_major=1).view(ctx.xshape)
        if ctx.needs_input_grad[1]:
            dw = K.gemm(dy2, x2, a_major=1, b_major=1)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy2.float().sum(0).to(dy2.dtype)
        return dx, dw, db, None


def _gemm_ok(x, w):
    return x.shape[-1] % 8 == 0 and w.shape[0] % 8 == 0 and x.numel() > 0


def _tc_other(*ts) -> bool:
    """fp16 tensors, or fp32 tensors while TF32 is enabled (`lt.cuda.set_tf32_enabled`, on by default as in the
    reference), on a CUDA device: they run on the same tcgen05 GEMM as bf16 (`kernels.gemm_any`)."""
    from .. import cuda as _cuda
    dt = None
    for t in ts:
        if t is None:
            continue
        if not t.is_cuda or t.dtype not in (torch.float16, torch.float32) or (dt is not None and t.dtype != dt):
            return False
        dt = t.dtype
    return dt == torch.float16 or (dt == torch.float32 and _cuda.is_tf32_enabled())


class _LinearAny(torch.autograd.Function):
    """y = x @ w^T (+ b) for fp16 / fp32 (tf32) CUDA tensors on the tcgen05 GEMM; same three GEMMs as `_Linear`."""

    @staticmethod
    def forward(ctx, x, w, b):
        x2 = _2d(x).contiguous()
        wc = w.contiguous()
        y = K.gemm_any(x2, wc)
        if b is not None:
            y = y + b
        ctx.save_for_backward(x2, wc)
        ctx.has_bias = b is not None
        ctx.xshape = x.shape
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = _2d(dy).contiguous()
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = K.gemm_any(dy2, w, b_major=1).view(ctx.xshape)
        if ctx.needs_input_grad[1]:
            dw = K.gemm_any(dy2, x2, a_major=1, b_major=1)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy2.float().sum(0).to(dy2.dtype)
        return dx, dw, db


class _MatmulAny(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, b):
        a, b = a.contiguous(), b.contiguous()
        ctx.save_for_backward(a, b)
        return K.gemm_any(a, b, b_major=1)

    @staticmethod
    def backward(ctx, dc):
        a, b = ctx.saved_tensors
        dc = dc.contiguous()
        da = K.gemm_any(dc, b) if ctx.needs_input_grad[0] else None
        db = K.gemm_any(a, dc, a_major=1, b_major=1) if ctx.needs_input_grad[1] else None
        return da, db


def bmm(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """[B, M, K] @ [B, K, N] on the tcgen05 GEMM, one launch per batch entry (CUDA bf16 / fp16 / tf32 with dimensions
    that are multiples of 8); `torch.bmm` elsewhere.  Reference: cublasSgemmStridedBatched
    (src/backend/gpu_native/math/gemm.cu:49-73)."""
    ok = (a.dim() == 3 and b.dim() == 3 and a.shape[0] == b.shape[0] and a.shape[0] <= 64 and a.shape[-1] % 8 == 0
          and b.shape[-1] % 8 == 0 and a.shape[1] % 8 == 0 and a.numel() > 0 and b.numel() > 0)
    if ok and (_native(a, b) or _tc_other(a, b)):
        fn = _MatmulNN if a.dtype == torch.bfloat16 else _MatmulAny
        return torch.stack([fn.apply(a[i], b[i]) for i in range(a.shape[0])], 0)
    return torch.bmm(a, b)


def linear(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor] = None, act: str = "none") -> torch.Tensor:
    """y = act(x @ w^T + b), w: [out, in]."""
    code = {"none": 0, "gelu": 1}[act]
    if _native(x, w, b) and _gemm_ok(x, w):
        return _Linear.apply(x, w, b, code)
    if _tc_other(x, w, b) and _gemm_ok(x, w) and w.shape[1] % 8 == 0:
        y = _LinearAny.apply(x, w, b)
        return F.gelu(y, approximate="tanh") if code == 1 else y
    y = F.linear(x, w, b)
    return F.gelu(y, approximate="tanh") if code == 1 else y


class _LinearFP8(torch.autograd.Function):
    """y = x @ w^T with e4m3 operands: 1 x 128 scales on the activations (and on dY), 128 x 128 scales on the weight
    (and on its transpose for the input gradient); the weight gradient stays in bf16.  Master weights are bf16."""

    @staticmethod
    def forward(ctx, x, w):
        x2 = _2d(x).contiguous()
        xq, xs = K.quant_fp8_1x128(x2)
        wq, ws = K.quant_fp8_128x128(w.contiguous())
        y = K.gemm_fp8_block(xq, xs, wq, ws)
        ctx.save_for_backward(x2, w)
        ctx.xshape = x.shape
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = _2d(dy).contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            gq, gs = K.quant_fp8_1x128(dy2)
            wtq, wts = K.quant_fp8_128x128(w.t().contiguous())      # [K, N]: the B operand of dX = dY @ W
            dx = K.gemm_fp8_block(gq, gs, wtq, wts).view(ctx.xshape)
        if ctx.needs_input_grad[1]:
            dw = K.gemm(dy2, x2, a_major=1, b_major=1)
        return dx, dw


class _LinearFP8Rows(torch.autograd.Function):
    """y = x @ w^T with e4m3 operands scaled per row: one scale per token for the activations (and for dY), one per output
    channel for the weight (per input channel for its transpose in the input gradient).  The products accumulate over the
    whole K extent in tensor memory and the scales are applied once in the epilogue (`K.gemm_e4m3`), which is what lets this
    path run faster than bf16; the weight gradient stays in bf16.  Master weights are bf16."""

    @staticmethod
    def forward(ctx, x, w):
        x2 = _2d(x).contiguous()
        xq, xs = K.quant_e4m3_rows(x2)
        wq, ws = K.quant_e4m3_rows(w.contiguous())
        y = K.gemm_e4m3(xq, xs, wq, ws)
        ctx.save_for_backward(x2, w)
        ctx.xshape = x.shape
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = _2d(dy).contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            gq, gs = K.quant_e4m3_rows(dy2)
            wtq, wts = K.quant_e4m3_rows(w.t().contiguous())      # [K, N]: the B operand of dX = dY @ W, scaled per input channel
            dx = K.gemm_e4m3(gq, gs, wtq, wts).view(ctx.xshape)
        if ctx.needs_input_grad[1]:
            dw = K.gemm(dy2, x2, a_major=1, b_major=1)
        return dx, dw


def linear_fp8(x: torch.Tensor, w: torch.Tensor, scaling: str = "rows") -> torch.Tensor:
    """Linear layer with e4m3 operands on the tensor cores (forward and input gradient; the weight gradient stays bf16).
    scaling="rows" (default): one scale per token and per channel, applied in the GEMM epilogue - the fast path;
    scaling="block": 1 x 128 / 128 x 128 block scales with two-level accumulation (feature dimensions multiples of 128).
    Falls back to `linear` where the shapes do not fit."""
    ok = _native(x, w) and x.dtype == torch.bfloat16 and x.numel() > 0
    if ok and scaling == "rows" and x.shape[-1] % 16 == 0 and w.shape[0] % 16 == 0:
        return _LinearFP8Rows.apply(x, w)
    if ok and scaling == "block" and x.shape[-1] % 128 == 0 and w.shape[0] % 128 == 0:
        return _LinearFP8.apply(x, w)
    return linear(x, w)


class _MatmulNN(torch.autograd.Function):
    """C = A[M,K] @ B[K,N] for 2-D bf16 CUDA operands."""

    @staticmethod
    def forward(ctx, a, b):
        a, b = a.contiguous(), b.contiguous()
        ctx.save_for_backward(a, b)
        return K.gemm(a, b, b_major=1)

    @staticmethod
    def backward(ctx, dc):
        a, b = ctx.saved_tensors
        dc = dc.contiguous()
        da = K.gemm(dc, b) if ctx.needs_input_grad[0] else None                       # dC[M,N] @ B[K,N]^T
        db = K.gemm(a, dc, a_major=1, b_major=1) if ctx.needs_input_grad[1] else None  # A^T @ dC
        return da, db


def matmul(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    if (_native(a, b) and b.dim() == 2 and a.shape[-1] % 8 == 0 and b.shape[-1] % 8 == 0 and a.numel() > 0 and
            b.numel() > 0):
        out = _MatmulNN.apply(_2d(a), b)
        return out.view(*a.shape[:-1], b.shape[-1])
    if (_tc_other(a, b) and b.dim() == 2 and a.dim() >= 2 and a.shape[-1] % 8 == 0 and b.shape[-1] % 8 == 0 and a.numel() > 0
            and b.numel() > 0 and _2d(a).shape[0] % 8 == 0):
        out = _MatmulAny.apply(_2d(a), b)
        return out.view(*a.shape[:-1], b.shape[-1])
    return torch.matmul(a, b)


# ---------------------------------------------------------------------------------------------- norms
class _Norm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, b, residual, eps, layer_norm):
        x2 = _2d(x).contiguous()
        r2 = _2d(residual).contiguous() if residual is not None else None
        y, s, mean, rstd = K.norm_fwd(x2, w.contiguous(), b.contiguous() if b is not None else None, r2,
                                      layer_norm=layer_norm, eps=eps)
        xin = s if r2 is not None else x2
        ctx.save_for_backward(xin, w, mean, rstd)
        ctx.layer_norm = layer_norm
        ctx.has_res = r2 is not None
        ctx.has_bias = b is not None
        ctx.shape = x.shape
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        xin, w, mean, rstd = ctx.saved_tensors
        dx, dw, db = K.norm_bwd(_2d(dy).contiguous(), xin, w.contiguous(), mean, rstd, layer_norm=ctx.layer_norm)
        dx = dx.view(ctx.shape)
        return dx, dw, (db if ctx.has_bias else None), (dx if ctx.has_res else None), None, None


def _norm_ok(x):
    return x.shape[-1] % 8 == 0 and x.shape[-1] <= 16384 and x.numel() > 0


def rms_norm(x, w, eps: float = 1e-5, residual=None):
    if _native(x, w, residual) and _norm_ok(x):
        return _Norm.apply(x, w, None, residual, eps, False)
    xs = x if residual is None else x + residual
    xf = xs.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * w


def layer_norm(x, w, b, eps: float = 1e-5, residual=None):
    if _native(x, w, b, residual) and _norm_ok(x) and b is not None:
        return _Norm.apply(x, w, b, residual, eps, True)
    xs = x if residual is None else x + residual
    return F.layer_norm(xs, (x.shape[-1],), w, b, eps)


# ---------------------------------------------------------------------------------------------- activations
class _Gelu(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        xc = x.contiguous()
        ctx.save_for_backward(xc)
        return K.gelu_fwd(xc)

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        return K.gelu_bwd(x, dy.contiguous())


def gelu(x):
    if _native(x) and x.numel() % 8 == 0 and x.numel() > 0:
        return _Gelu.apply(x)
    return F.gelu(x, approximate="tanh")


class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        g2 = _2d(gu).contiguous()
        ctx.save_for_backward(g2)
        ctx.shape = gu.shape
        return K.swiglu_fwd(g2).view(*gu.shape[:-1], gu.shape[-1] // 2)

    @staticmethod
    def backward(ctx, dh):
        (g2,) = ctx.saved_tensors
        return K.swiglu_bwd(g2, _2d(dh).contiguous(), inplace=False).view(ctx.shape)


def swiglu(gu):
    """gu = [..., 2F] with the gate in the first half: silu(gate) * up."""
    if _native(gu) and gu.shape[-1] % 16 == 0 and gu.numel() > 0:
        return _SwiGLU.apply(gu)
    f = gu.shape[-1] // 2
    return F.silu(gu[..., :f]) * gu[..., f:]


# ---------------------------------------------------------------------------------------------- RoPE
def _rope_torch(x, cos, sin, sign=1.0):
    # x: [B, H, T, D] with interleaved pairs; cos/sin: [T, D/2]
    T = x.shape[-2]
    c = cos[:T].to(x.dtype)
    s = (sin[:T] * sign).to(x.dtype)
    x0, x1 = x[..., 0::2], x[..., 1::2]
    return torch.stack([x0 * c - x1 * s, x0 * s + x1 * c], dim=-1).flatten(-2)


class _Rope(torch.autograd.Function):
    """x: [B, H, T, D] (reference layout, src/ops/rope.cpp:25-84)."""

    @staticmethod
    def forward(ctx, x, cos, sin):
        B, H, T, D = x.shape
        y = x.transpose(1, 2).contiguous()  # [B, T, H, D]
        K.rope_(y.view(B * T, H * D), cos, sin, T, H, D)
        ctx.save_for_backward(cos, sin)
        return y.transpose(1, 2)

    @staticmethod
    def backward(ctx, dy):
        cos, sin = ctx.saved_tensors
        B, H, T, D = dy.shape
        g = dy.transpose(1, 2).contiguous()
        K.rope_(g.view(B * T, H * D), cos, sin, T, H, D, backward=True)
        return g.transpose(1, 2), None, None


def rope(x, cos, sin):
    if _native(x) and x.dim() == 4 and x.shape[-1] % 8 == 0 and cos.is_cuda:
        return _Rope.apply(x, cos.float().contiguous(), sin.float().contiguous())
    return _rope_torch(x, cos, sin)


class _RopeBTHD(torch.autograd.Function):
    """x: [B, T, H, D], the layout of the fused QKV projection: rotated on a copy, no transposes."""

    @staticmethod
    def forward(ctx, x, cos, sin):
        B, T, H, D = x.shape
        y = x.contiguous().clone()
        K.rope_(y.view(B * T, H * D), cos, sin, T, H, D)
        ctx.save_for_backward(cos, sin)
        return y

    @staticmethod
    def backward(ctx, dy):
        cos, sin = ctx.saved_tensors
        B, T, H, D = dy.shape
        g = dy.contiguous().clone()
        K.rope_(g.view(B * T, H * D), cos, sin, T, H, D, backward=True)
        return g, None, None


def rope_bthd(x, cos, sin):
    """RoPE on [B, T, H, D] (interleaved pairs, cos/sin [T, D/2])."""
    if _native(x) and x.dim() == 4 and x.shape[-1] % 8 == 0 and cos.is_cuda:
        return _RopeBTHD.apply(x, cos.float().contiguous(), sin.float().contiguous())
    return _rope_torch(x.transpose(1, 2), cos, sin).transpose(1, 2)


# ---------------------------------------------------------------------------------------------- attention
class _Flash(torch.autograd.Function):
    """q: [B, Tq, Hq, D], k/v: [B, Tk, Hkv, D]."""

    @staticmethod
    def forward(ctx, q, k, v, causal, scale):
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        o, lse = K.flash_fwd(q, k, v, causal=causal, scale=scale)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.causal, ctx.scale = causal, scale
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse = ctx.saved_tensors
        dq, dk, dv = K.flash_bwd(q, k, v, o, lse, do.contiguous(), causal=ctx.causal, scale=ctx.scale)
        return dq, dk, dv, None, None


def flash_attention_bthd(q, k, v, causal: bool = False, scale: Optional[float] = None):
    """q: [B, Tq, Hq, D]; k, v: [B, Tk, Hkv, D]; Hq a multiple of Hkv."""
    D = q.shape[-1]
    scale = (D ** -0.5) if scale is None else scale
    if _native(q, k, v) and D in (64, 128) and q.shape[2] % k.shape[2] == 0:
        return _Flash.apply(q, k, v, bool(causal), float(scale))
    qh, kh, vh = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
    G = qh.shape[1] // kh.shape[1]
    if G > 1:
        kh, vh = kh.repeat_interleave(G, 1), vh.repeat_interleave(G, 1)
    s = torch.matmul(qh.float(), kh.float().transpose(-1, -2)) * scale
    if causal:
        Tq, Tk = s.shape[-2], s.shape[-1]
        i = torch.arange(Tq, device=s.device)[:, None] + (Tk - Tq)
        j = torch.arange(Tk, device=s.device)[None, :]
        s = s.masked_fill(j > i, float("-inf"))
    o = torch.matmul(torch.softmax(s, -1), vh.float()).to(q.dtype)
    return o.transpose(1, 2)


def flash_attention(q, k, v, is_causal: bool = False, scale: Optional[float] = None):
    """Reference layout [B, H, T, D] (src/ops/attention.cpp:187-349), with the causal flag its README documents."""
    return flash_attention_bthd(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal, scale).transpose(1, 2)


# ---------------------------------------------------------------------------------------------- losses / embedding
class _CrossEntropy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, targets, ignore_index):
        work = logits.contiguous().clone()
        tgt = targets.to(torch.int64).contiguous()
        n_valid = int((tgt != ignore_index).sum().item())
        stats = K.ce_stats(work, tgt)
        rows = K.ce_finish(work, tgt, stats, grad_scale=1.0 / max(n_valid, 1), ignore_index=ignore_index)
        ctx.save_for_backward(work)
        return (rows.sum() / max(n_valid, 1)).to(torch.float32)

    @staticmethod
    def backward(ctx, dl):
        (dlogits,) = ctx.saved_tensors
        return dlogits * dl.to(dlogits.dtype), None, None


def cross_entropy(logits, targets, ignore_index: int = -100):
    """Mean cross-entropy of logits [N, C] against class indices [N] (float or integer tensor)."""
    if _native(logits) and logits.dim() == 2:
        return _CrossEntropy.apply(logits, targets, ignore_index)
    return F.cross_entropy(logits.float(), targets.to(torch.int64), ignore_index=ignore_index)


class _Embedding(torch.autograd.Function):
    @staticmethod
    def forward(ctx, idx, table):
        idx64 = idx.to(torch.int64).contiguous()
        ctx.save_for_backward(idx64)
        ctx.tshape = table.shape
        return K.embedding_fwd(idx64, table.contiguous()).view(*idx.shape, table.shape[1])

    @staticmethod
    def backward(ctx, dout):
        (idx,) = ctx.saved_tensors
        dt = torch.zeros(ctx.tshape, dtype=dout.dtype, device=dout.device)
        K.embedding_bwd(idx, dout.reshape(-1, ctx.tshape[1]).contiguous(), dt)
        return None, dt


def embedding(idx, table):
    if _native(table) and table.shape[1] % 8 == 0 and idx.is_cuda:
        return _Embedding.apply(idx, table)
    return F.embedding(idx.to(torch.int64), table)


# ------------------------------------------------------------------------------------------------ softmax / dropout / router
class _Softmax(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        y = K.softmax_fwd(x)
        ctx.save_for_backward(y)
        return y

    @staticmethod
    def backward(ctx, dy):
        (y,) = ctx.saved_tensors
        return K.softmax_bwd(y, dy.contiguous())


def softmax(x: torch.Tensor, dim: int = -1) -> torch.Tensor:
    """Softmax over `dim`; the last-dimension case of fp32 / bf16 CUDA tensors runs on the warp-per-row kernel
    (reference: Ops::softmax, src/ops/activation.cpp:507-578)."""
    if _native(x) and x.dtype in (torch.float32, torch.bfloat16) and dim in (-1, x.dim() - 1) and x.numel() > 0:
        return _Softmax.apply(x.contiguous())
    return torch.softmax(x, dim)


_dropout_offset = [0]


class _Dropout(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, p, seed, offset):
        ctx.p, ctx.seed, ctx.offset = p, seed, offset
        return K.dropout(x, p, seed, offset)

    @staticmethod
    def backward(ctx, dy):
        return K.dropout(dy.contiguous(), ctx.p, ctx.seed, ctx.offset), None, None, None


def dropout(x: torch.Tensor, p: float, training: bool = True) -> torch.Tensor:
    """Inverted dropout. On CUDA the mask comes from a Philox counter keyed by torch's seed and a running offset, and
    backward regenerates it instead of storing it (reference: nn::Dropout, src/nn/dropout.cpp, which keeps a mask)."""
    if not training or p <= 0.0:
        return x
    if _native(x) and x.dtype in (torch.float32, torch.bfloat16):
        seed = torch.initial_seed()
        offset = _dropout_offset[0]
        _dropout_offset[0] += (x.numel() + 3) // 4
        return _Dropout.apply(x.contiguous(), float(p), seed, offset)
    return torch.nn.functional.dropout(x, p, True)


class _Router(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, top_k, renorm):
        probs, tw, ti = K.moe_router(logits, top_k, renorm=renorm)
        ctx.save_for_backward(probs, tw, ti)
        ctx.renorm = renorm
        ctx.in_dtype = logits.dtype
        ctx.mark_non_differentiable(ti)
        return tw, ti, probs

    @staticmethod
    def backward(ctx, d_tw, d_ti, d_probs):
        probs, tw, ti = ctx.saved_tensors
        if d_tw is None:
            d_tw = torch.zeros_like(tw)
        dl = K.moe_router_bwd(probs, ti, tw, d_tw, d_probs, renorm=ctx.renorm)
        return dl.to(ctx.in_dtype), None, None


def moe_router(logits: torch.Tensor, top_k: int, renorm: bool = True):
    """(top-k weights [N, k] fp32, expert ids [N, k], softmax probabilities [N, E] fp32) of router logits [N, E];
    the warp-per-token kernel on CUDA when E <= 256 and k <= 8 (reference: Ops::moe_gate, src/ops/moe_ops.cpp:11-106)."""
    if _native(logits) and logits.dtype in (torch.float32, torch.bfloat16) and logits.shape[1] <= 256 and top_k <= 8:
        tw, ti, probs = _Router.apply(logits.contiguous(), top_k, renorm)
        return tw, ti.long(), probs
    probs = torch.softmax(logits.float(), -1)
    top_p, top_i = probs.topk(top_k, -1)
    if renorm:
        top_p = top_p / top_p.sum(-1, keepdim=True)
    return top_p, top_i, probs


class _FusedLinearCE(torch.autograd.Function):
    """Mean cross-entropy of x @ W^T against integer targets without ever holding the [N, V] logits: rows go through in
    chunks, and because the gradient of the loss with respect to the logits needs nothing from upstream but one scalar,
    each chunk's logits are turned into their gradient in place (`lt_ce_finish`) and consumed at once by the two
    gradient GEMMs - d(x) for the chunk and the running d(W).  Backward only scales the two stored gradients.  The
    reference chunks the same way but recomputes the logits in backward (src/ops/fused_loss.cpp:12-195)."""

    @staticmethod
    def forward(ctx, x, w, target, chunk_rows):
        from . import kernels as K
        N, Kd = x.shape
        V = w.shape[0]
        tgt = target.to(torch.int64).contiguous()
        x = x.contiguous()
        w = w.contiguous()
        n_chunks = (N + chunk_rows - 1) // chunk_rows
        dx = torch.empty_like(x)
        dw = torch.empty((V, Kd), dtype=torch.float32 if n_chunks > 4 else torch.bfloat16, device=x.device)
        total = torch.zeros((), dtype=torch.float32, device=x.device)
        for ci, s0 in enumerate(range(0, N, chunk_rows)):
            xc, tc = x[s0:s0 + chunk_rows], tgt[s0:s0 + chunk_rows]
            logits = K.gemm(xc, w)                                    # [chunk, V]: the only piece of the logits that exists
            stats = K.ce_stats(logits, tc)
            rows = K.ce_finish(logits, tc, stats, grad_scale=1.0 / N)  # logits now hold d(loss)/d(logits)
            total = total + rows.sum()
            K.gemm(logits, w, b_major=1, out=dx[s0:s0 + chunk_rows])
            K.gemm(logits, xc, a_major=1, b_major=1, out=dw, accumulate=ci > 0)
        ctx.save_for_backward(dx, dw)
        ctx.w_dtype = w.dtype
        return total / N

    @staticmethod
    def backward(ctx, g):
        dx, dw = ctx.saved_tensors
        return dx * g.to(dx.dtype), (dw * g).to(ctx.w_dtype), None, None


def fused_linear_cross_entropy(x: torch.Tensor, w: torch.Tensor, target: torch.Tensor, chunk_rows: int = 4096):
    """Kernel path of `Ops.fused_linear_cross_entropy` (CUDA, bf16, no bias); None when it does not apply."""
    if not (_native(x) and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.dim() == 2 and w.is_cuda):
        return None
    return _FusedLinearCE.apply(x, w, target, int(chunk_rows))
