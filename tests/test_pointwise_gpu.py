"""Norm / RoPE / SwiGLU / GELU / embedding / cross-entropy / AdamW kernels against fp32 PyTorch."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _close(a, b, tol):
    err = ((a.float() - b.float()).norm() / (b.float().norm() + 1e-6)).item()
    assert err < tol, err


@pytest.mark.parametrize("layer_norm", [False, True])
@pytest.mark.parametrize("M,D", [(64, 2048), (37, 512), (5, 4096), (700, 128)])
def test_norm_fwd_bwd(layer_norm, M, D):
    from litetorch_b200.ops import kernels as K
    torch.manual_seed(0)
    x = torch.randn(M, D, device="cuda").bfloat16()
    r = torch.randn(M, D, device="cuda").bfloat16()
    w = (1 + 0.1 * torch.randn(D, device="cuda")).bfloat16()
    b = (0.1 * torch.randn(D, device="cuda")).bfloat16() if layer_norm else None
    dy = torch.randn(M, D, device="cuda").bfloat16()
    y, s, mean, rstd = K.norm_fwd(x, w, b, r, layer_norm=layer_norm, eps=1e-5)
    sf = (x.float() + r.float()).bfloat16().float().requires_grad_(True)
    wf = w.float().requires_grad_(True)
    if layer_norm:
        bf = b.float().requires_grad_(True)
        yr = torch.nn.functional.layer_norm(sf, (D,), wf, bf, 1e-5)
    else:
        yr = sf * torch.rsqrt(sf.pow(2).mean(-1, keepdim=True) + 1e-5) * wf
    _close(s, sf, 1e-3)
    _close(y, yr, 1e-2)
    yr.backward(dy.float())
    dx, dw, db = K.norm_bwd(dy, s, w, mean, rstd, layer_norm=layer_norm)
    _close(dx, sf.grad, 1.5e-2)
    _close(dw, wf.grad, 1.5e-2)
    if layer_norm:
        _close(db, bf.grad, 1.5e-2)
    y2, _, _, _ = K.norm_fwd(x, w, b, None, layer_norm=layer_norm)
    xf = x.float()
    if layer_norm:
        _close(y2, torch.nn.functional.layer_norm(xf, (D,), w.float(), b.float(), 1e-5), 1e-2)
    else:
        _close(y2, xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5) * w.float(), 1e-2)


def _rope_ref(x, cos, sin):
    # x: [rows(T-major), H, D] interleaved pairs
    T = cos.shape[0]
    rows, H, D = x.shape
    t = torch.arange(rows, device=x.device) % T
    c = cos[t][:, None, :]
    s = sin[t][:, None, :]
    x0, x1 = x[..., 0::2], x[..., 1::2]
    out = torch.empty_like(x)
    out[..., 0::2] = x0 * c - x1 * s
    out[..., 1::2] = x0 * s + x1 * c
    return out


def test_rope_roundtrip_and_ref():
    from litetorch_b200.ops import kernels as K
    torch.manual_seed(0)
    B, T, H, Hkv, D = 2, 48, 4, 2, 64
    pitch = (H + 2 * Hkv) * D
    qkv = torch.randn(B * T, pitch, device="cuda").bfloat16()
    orig = qkv.clone()
    inv = 1.0 / (10000 ** (torch.arange(0, D, 2, device="cuda").float() / D))
    ang = torch.arange(T, device="cuda").float()[:, None] * inv[None]
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    K.rope_(qkv, cos, sin, T, H, D, col_offset=0)
    K.rope_(qkv, cos, sin, T, Hkv, D, col_offset=H * D)
    ref_q = _rope_ref(orig[:, :H * D].float().view(B * T, H, D), cos, sin)
    ref_k = _rope_ref(orig[:, H * D:(H + Hkv) * D].float().view(B * T, Hkv, D), cos, sin)
    _close(qkv[:, :H * D].reshape(B * T, H, D), ref_q, 1e-2)
    _close(qkv[:, H * D:(H + Hkv) * D].reshape(B * T, Hkv, D), ref_k, 1e-2)
    assert torch.equal(qkv[:, (H + Hkv) * D:], orig[:, (H + Hkv) * D:])
    K.rope_(qkv, cos, sin, T, H, D, col_offset=0, backward=True)
    _close(qkv[:, :H * D], orig[:, :H * D], 2e-2)


def test_swiglu_gelu():
    from litetorch_b200.ops import kernels as K
    torch.manual_seed(0)
    M, F = 96, 1408
    gu = torch.randn(M, 2 * F, device="cuda").bfloat16()
    dh = torch.randn(M, F, device="cuda").bfloat16()
    h = K.swiglu_fwd(gu)
    guf = gu.float().requires_grad_(True)
    hr = torch.nn.functional.silu(guf[:, :F]) * guf[:, F:]
    _close(h, hr, 1e-2)
    hr.backward(dh.float())
    dgu = K.swiglu_bwd(gu.clone(), dh)
    _close(dgu, guf.grad, 1e-2)
    x = torch.randn(M, F, device="cuda").bfloat16()
    xf = x.float().requires_grad_(True)
    yr = torch.nn.functional.gelu(xf, approximate="tanh")
    _close(K.gelu_fwd(x), yr, 1e-2)
    yr.backward(dh.float())
    _close(K.gelu_bwd(x, dh), xf.grad, 1e-2)


def test_embedding():
    from litetorch_b200.ops import kernels as K
    torch.manual_seed(0)
    V, D, N = 1000, 256, 4096
    table = torch.randn(V, D, device="cuda").bfloat16()
    idx = torch.randint(0, V, (N,), device="cuda")
    out = K.embedding_fwd(idx, table)
    assert torch.equal(out, table[idx])
    dout = torch.randn(N, D, device="cuda").bfloat16()
    dt = torch.zeros(V, D, device="cuda").bfloat16()
    K.embedding_bwd(idx, dout, dt)
    ref = torch.zeros(V, D, device="cuda").index_add_(0, idx, dout.float())
    _close(dt, ref, 3e-2)


@pytest.mark.parametrize("N,V", [(64, 32000), (33, 1003), (8, 128256)])
def test_cross_entropy(N, V):
    from litetorch_b200.ops import kernels as K
    torch.manual_seed(0)
    logits = (torch.randn(N, V, device="cuda") * 2).bfloat16()
    tgt = torch.randint(0, V, (N,), device="cuda")
    tgt[0] = -100
    lf = logits.float().requires_grad_(True)
    ref = torch.nn.functional.cross_entropy(lf, tgt, ignore_index=-100, reduction="sum")
    ref.backward()
    stats = K.ce_stats(logits, tgt)
    work = logits.clone()
    loss = K.ce_finish(work, tgt, stats, grad_scale=1.0)
    assert abs(loss.sum().item() - ref.item()) / abs(ref.item()) < 2e-3
    _close(work, lf.grad, 2e-2)
    # two vocabulary shards combined like tensor-parallel ranks do
    h = (V // 2) // 8 * 8
    s0 = K.ce_stats(logits[:, :h], tgt, 0)
    s1 = K.ce_stats(logits[:, h:], tgt, h) if (h % 8 == 0 and logits[:, h:].data_ptr() % 16 == 0) else None
    if s1 is not None:
        gm = torch.maximum(s0[:, 0], s1[:, 0])
        gs = s0[:, 1] * torch.exp(s0[:, 0] - gm) + s1[:, 1] * torch.exp(s1[:, 0] - gm)
        g = torch.stack([gm, gs, s0[:, 2] + s1[:, 2]], 1).contiguous()
        _close(g[1:, 1].log() + g[1:, 0], stats[1:, 1].log() + stats[1:, 0], 1e-4)


def test_adamw_flat_matches_torch():
    from litetorch_b200.ops import kernels as K
    torch.manual_seed(0)
    n = 100003
    p = torch.randn(n, device="cuda")
    ref_p = p.clone().requires_grad_(True)
    opt = torch.optim.AdamW([ref_p], lr=3e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    m = torch.zeros_like(p)
    v = torch.zeros_like(p)
    p16 = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    for step in range(1, 4):
        g = torch.randn(n, device="cuda")
        ref_p.grad = g.clone()
        opt.step()
        K.adam_flat(p, g, m, v, p16, lr=3e-4, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.1, step=step)
    assert (p - ref_p.detach()).abs().max().item() < 1e-5
    _close(p16, p, 5e-3)
    stats = torch.zeros(2, device="cuda")
    K.sumsq(g, stats)
    assert abs(stats[0].item() - g.pow(2).sum().item()) / g.pow(2).sum().item() < 1e-4
