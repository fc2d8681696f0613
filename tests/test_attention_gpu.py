"""tcgen05 FlashAttention forward/backward against an fp32 PyTorch reference (causal, GQA, tails)."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(q, k, v, causal, scale):
    B, Tq, Hq, D = q.shape
    Tk, Hkv = k.shape[1], k.shape[2]
    G = Hq // Hkv
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(G, dim=1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(G, dim=1)
    s = qf @ kf.transpose(-1, -2) * scale
    if causal:
        i = torch.arange(Tq, device=q.device)[:, None] + (Tk - Tq)
        j = torch.arange(Tk, device=q.device)[None, :]
        s = s.masked_fill(j > i, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    o = torch.softmax(s, dim=-1) @ vf
    return o.permute(0, 2, 1, 3), lse


def _err(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-6)).item()


CASES = [
    (2, 256, 256, 4, 2, 64, True),
    (1, 384, 384, 2, 1, 128, True),
    (2, 200, 200, 4, 4, 64, True),
    (1, 128, 320, 2, 2, 128, True),
    (1, 256, 256, 8, 2, 64, False),
    (1, 1024, 1024, 4, 1, 128, True),
]


@pytest.mark.parametrize("B,Tq,Tk,Hq,Hkv,D,causal", CASES)
def test_flash_fwd_bwd(B, Tq, Tk, Hq, Hkv, D, causal):
    from litetorch_b200.ops import kernels as K
    torch.manual_seed(0)
    q = torch.randn(B, Tq, Hq, D, device="cuda").bfloat16()
    k = torch.randn(B, Tk, Hkv, D, device="cuda").bfloat16()
    v = torch.randn(B, Tk, Hkv, D, device="cuda").bfloat16()
    do = torch.randn(B, Tq, Hq, D, device="cuda").bfloat16()
    scale = 1.0 / math.sqrt(D)
    o, lse = K.flash_fwd(q, k, v, causal=causal, scale=scale)
    torch.cuda.synchronize()
    K.check_status()
    qf, kf, vf = (x.float().requires_grad_(True) for x in (q, k, v))
    o_ref, lse_ref = _ref(qf, kf, vf, causal, scale)
    assert _err(o, o_ref) < 1e-2
    assert (lse - lse_ref).abs().max().item() < 2e-2
    o_ref.backward(do.float())
    dq, dk, dv = K.flash_bwd(q, k, v, o, lse, do, causal=causal, scale=scale)
    torch.cuda.synchronize()
    K.check_status()
    assert _err(dv, vf.grad) < 2e-2
    assert _err(dk, kf.grad) < 2e-2
    assert _err(dq, qf.grad) < 2e-2


def test_flash_strided_qkv_buffer():
    """q/k/v as column slices of one fused [B*T, (Hq+2Hkv)*D] projection output."""
    from litetorch_b200.ops import kernels as K
    torch.manual_seed(1)
    B, T, Hq, Hkv, D = 2, 256, 4, 2, 64
    pitch = (Hq + 2 * Hkv) * D
    buf = torch.randn(B, T, pitch, device="cuda").bfloat16()
    q = buf[:, :, :Hq * D].view(B, T, Hq, D)
    k = buf[:, :, Hq * D:(Hq + Hkv) * D].view(B, T, Hkv, D)
    v = buf[:, :, (Hq + Hkv) * D:].view(B, T, Hkv, D)
    o, lse = K.flash_fwd(q, k, v, causal=True)
    o_ref, _ = _ref(q, k, v, True, D ** -0.5)
    assert _err(o, o_ref) < 1e-2
    K.check_status()
