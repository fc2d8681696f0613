"""Plain-PyTorch twins of the kernel front-end in `kernels.py`, with the same names, arguments and in-place effects.

`LlamaEngine` and the weight providers pick this module when their tensors live on the CPU, so that the
hand-written forward/backward schedule, the sharding layouts and the collective logic run as gloo ranks in the
test-suite without a GPU (the reference tests its distributed code the same way, by forking CPU ranks:
tests/distributed_test.cpp).  Nothing here is used on a CUDA device.  Arithmetic is done in fp32 and rounded to
the dtype of the output buffer, which is what the kernels do.
"""
from __future__ import annotations

import math

import torch

_launches = [0]


def launch_count() -> int:
    return 0


def reset_launch_count():
    pass


def status_fetch() -> int:
    return 0


def check_status():
    pass


def gemm(a, b, *, a_major=0, b_major=0, out=None, out_dtype=None, bias=None, residual=None, act=0, accumulate=False,
         alpha=1.0, block_n=0, max_ctas=0):
    A = a.float() if a_major == 0 else a.float().t()
    B = b.float().t() if b_major == 0 else b.float()
    y = (A @ B) * alpha
    if bias is not None:
        y = y + bias.float()
    if act == 1:
        y = torch.nn.functional.gelu(y, approximate="tanh")
    if residual is not None:
        y = y + residual.float()
    if out is None:
        return y.to(out_dtype or a.dtype)
    if accumulate:
        out.copy_((out.float() + y).to(out.dtype))
    else:
        out.copy_(y.to(out.dtype))
    return out


def norm_fwd(x, weight, bias=None, residual=None, *, layer_norm=False, eps=1e-5, want_sum=True, out=None):
    xf = x.float()
    s = None
    if residual is not None:
        xf = xf + residual.float()
        s = xf.to(x.dtype) if want_sum else None
        xf = xf.to(x.dtype).float()
    mean = None
    if layer_norm:
        mean = xf.mean(-1)
        xc = xf - mean[:, None]
    else:
        xc = xf
    rstd = torch.rsqrt(xc.pow(2).mean(-1) + eps)
    y = xc * rstd[:, None] * weight.float()
    if bias is not None:
        y = y + bias.float()
    if out is not None:
        out.copy_(y.to(x.dtype))
        return out, s, mean, rstd
    return y.to(x.dtype), s, mean, rstd


def norm_bwd(dy, x, weight, mean, rstd, *, layer_norm=False, dres=None, dw=None, db=None, accumulate=False, out=None):
    xf, g = x.float(), dy.float()
    xc = xf - mean[:, None] if layer_norm else xf
    xhat = xc * rstd[:, None]
    gw = g * weight.float()
    D = x.shape[1]
    if layer_norm:
        dx = (gw - gw.mean(-1, keepdim=True) - xhat * (gw * xhat).mean(-1, keepdim=True)) * rstd[:, None]
    else:
        dx = (gw - xhat * (gw * xhat).sum(-1, keepdim=True) / D) * rstd[:, None]
    if dres is not None:
        dx = dx + dres.float()
    dwv = (g * xhat).sum(0)
    if dw is None:
        dw = dwv.to(weight.dtype)
    elif accumulate:
        dw.copy_((dw.float() + dwv).to(dw.dtype))
    else:
        dw.copy_(dwv.to(dw.dtype))
    if layer_norm:
        dbv = g.sum(0)
        if db is None:
            db = dbv.to(weight.dtype)
        elif accumulate:
            db.copy_((db.float() + dbv).to(db.dtype))
        else:
            db.copy_(dbv.to(db.dtype))
    if out is not None:
        out.copy_(dx.to(x.dtype))
        return out, dw, db
    return dx.to(x.dtype), dw, db


def rope_(x2d, cos, sin, T, heads, head_dim, *, col_offset=0, positions=None, backward=False):
    rows = x2d.shape[0]
    pos = positions.to(torch.int64) if positions is not None else torch.arange(rows, device=x2d.device) % T
    c = cos[pos][:, None, :]
    s = sin[pos][:, None, :]
    if backward:
        s = -s
    blk = x2d[:, col_offset:col_offset + heads * head_dim].float().reshape(rows, heads, head_dim // 2, 2)
    x0, x1 = blk[..., 0], blk[..., 1]
    out = torch.stack([x0 * c - x1 * s, x0 * s + x1 * c], dim=-1).reshape(rows, heads * head_dim)
    x2d[:, col_offset:col_offset + heads * head_dim] = out.to(x2d.dtype)
    return x2d


def swiglu_fwd(gu):
    F = gu.shape[1] // 2
    g, u = gu[:, :F].float(), gu[:, F:].float()
    return (torch.nn.functional.silu(g) * u).to(gu.dtype)


def swiglu_bwd(gu, dh, inplace=True):
    F = gu.shape[1] // 2
    g, u, d = gu[:, :F].float(), gu[:, F:].float(), dh.float()
    sg = torch.sigmoid(g)
    dg = d * u * (sg + g * sg * (1 - sg))
    du = d * g * sg
    out = gu if inplace else torch.empty_like(gu)
    out[:, :F] = dg.to(gu.dtype)
    out[:, F:] = du.to(gu.dtype)
    return out


def embedding_fwd(idx, table):
    idx = idx.reshape(-1).to(torch.int64).clamp(0, table.shape[0] - 1)
    return table[idx].contiguous()


def embedding_bwd(idx, dout, dtable):
    idx = idx.reshape(-1).to(torch.int64)
    ok = (idx >= 0) & (idx < dtable.shape[0])
    acc = dtable.float()
    acc.index_add_(0, idx[ok], dout[ok].float())
    dtable.copy_(acc.to(dtable.dtype))
    return dtable


def ce_stats(logits, targets, vocab_start=0):
    lf = logits.float()
    V = lf.shape[1]
    m = lf.amax(-1)
    s = torch.exp(lf - m[:, None]).sum(-1)
    loc = targets.to(torch.int64) - vocab_start
    inside = (loc >= 0) & (loc < V)
    tl = torch.where(inside, lf.gather(1, loc.clamp(0, V - 1)[:, None])[:, 0], torch.zeros_like(m))
    return torch.stack([m, s, tl], 1).contiguous()


def ce_finish(logits, targets, gstats, *, vocab_start=0, grad_scale=1.0, ignore_index=-100, write_grad=True):
    N, V = logits.shape
    tgt = targets.to(torch.int64)
    valid = tgt != ignore_index
    rows = torch.where(valid, torch.log(gstats[:, 1]) + gstats[:, 0] - gstats[:, 2], torch.zeros_like(gstats[:, 0]))
    if write_grad:
        p = torch.exp(logits.float() - gstats[:, 0:1]) / gstats[:, 1:2]
        loc = tgt - vocab_start
        inside = (loc >= 0) & (loc < V) & valid
        p[torch.arange(N, device=p.device)[inside], loc[inside]] -= 1.0
        p = p * valid[:, None] * grad_scale
        logits.copy_(p.to(logits.dtype))
    return rows


def _expand_kv(k, Hq):
    B, T, Hkv, D = k.shape
    return k if Hkv == Hq else k[:, :, :, None, :].expand(B, T, Hkv, Hq // Hkv, D).reshape(B, T, Hq, D)


def flash_fwd(q, k, v, *, causal=True, scale=None):
    B, Tq, Hq, D = q.shape
    Tk = k.shape[1]
    scale = (D ** -0.5) if scale is None else scale
    qf = q.float().permute(0, 2, 1, 3)
    kf = _expand_kv(k.float(), Hq).permute(0, 2, 1, 3)
    vf = _expand_kv(v.float(), Hq).permute(0, 2, 1, 3)
    s = qf @ kf.transpose(-1, -2) * scale
    if causal:
        mask = torch.ones(Tq, Tk, dtype=torch.bool, device=q.device).tril(Tk - Tq)
        s = s.masked_fill(~mask, float("-inf"))
    lse = torch.logsumexp(s, -1)
    o = torch.exp(s - lse[..., None]) @ vf
    return o.permute(0, 2, 1, 3).contiguous().to(q.dtype), lse.contiguous()


def flash_bwd(q, k, v, o, lse, do, *, causal=True, scale=None, dq=None, dk=None, dv=None):
    B, Tq, Hq, D = q.shape
    _, Tk, Hkv, _ = k.shape
    scale = (D ** -0.5) if scale is None else scale
    qf = q.float().permute(0, 2, 1, 3)
    kf = _expand_kv(k.float(), Hq).permute(0, 2, 1, 3)
    vf = _expand_kv(v.float(), Hq).permute(0, 2, 1, 3)
    dof = do.float().permute(0, 2, 1, 3)
    of = o.float().permute(0, 2, 1, 3)
    s = qf @ kf.transpose(-1, -2) * scale
    if causal:
        mask = torch.ones(Tq, Tk, dtype=torch.bool, device=q.device).tril(Tk - Tq)
        s = s.masked_fill(~mask, float("-inf"))
    p = torch.exp(s - lse[..., None])
    dvf = p.transpose(-1, -2) @ dof
    dp = dof @ vf.transpose(-1, -2)
    delta = (dof * of).sum(-1, keepdim=True)
    ds = p * (dp - delta) * scale
    dqf = ds @ kf
    dkf = ds.transpose(-1, -2) @ qf
    g = Hq // Hkv
    dkf = dkf.reshape(B, Hkv, g, Tk, D).sum(2)
    dvf = dvf.reshape(B, Hkv, g, Tk, D).sum(2)
    res = []
    for buf, val in ((dq, dqf), (dk, dkf), (dv, dvf)):
        val = val.permute(0, 2, 1, 3)
        if buf is None:
            res.append(val.contiguous().to(q.dtype))
        else:
            buf.copy_(val.to(buf.dtype))
            res.append(buf)
    return tuple(res)


def adam_flat(master, grad, m, v, param_bf16, *, lr, beta1, beta2, eps, wd, step, adamw=True, dyn=None):
    g = grad.float()
    if dyn is not None:
        if float(dyn[1]) != 0.0:
            return
        g = g * float(dyn[0])
    bc1 = 1.0 - beta1 ** step
    bc2 = 1.0 - beta2 ** step
    if not adamw and wd != 0.0:
        g = g + wd * master
    m.mul_(beta1).add_(g, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    if adamw:
        master.mul_(1.0 - lr * wd)
    master.addcdiv_(m / bc1, (v / bc2).sqrt() + eps, value=-lr)
    if param_bf16 is not None:
        param_bf16.copy_(master.to(param_bf16.dtype))


def sumsq(x, out):
    out[0] += x.float().pow(2).sum()
    out[1] += (~torch.isfinite(x.float())).sum()
    return out


def clip_coef(stats, dyn, max_norm, inv_scale=1.0):
    norm = math.sqrt(float(stats[0])) * inv_scale
    coef = min(1.0, max_norm / (norm + 1e-6)) if max_norm > 0 else 1.0
    dyn[0] = coef * inv_scale
    dyn[1] = 1.0 if float(stats[1]) != 0.0 else 0.0
    dyn[2] = norm
    return dyn
