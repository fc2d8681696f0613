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


def _ref_rows(q, k, v, do, rows, scale):
    """fp32 causal attention forward restricted to the query rows `rows` of one (batch, head): (o, lse) there, plus the
    contribution of those rows to dK / dV and their dQ (enough to check a long sequence without a T x T matrix)."""
    qf, kf, vf, dof = q.float(), k.float(), v.float(), do.float()          # [T, D] each; qf / dof indexed by rows
    s = qf[rows] @ kf.t() * scale
    j = torch.arange(kf.shape[0], device=q.device)[None, :]
    s = s.masked_fill(j > rows[:, None], float("-inf"))
    lse = torch.logsumexp(s, -1)
    p = torch.exp(s - lse[:, None])
    o = p @ vf
    dp = dof[rows] @ vf.t()
    delta = (dof[rows] * o).sum(-1, keepdim=True)
    ds = p * (dp - delta) * scale
    return o, lse, ds @ kf


@pytest.mark.parametrize("B,T,Hq,Hkv,D", [(4, 2048, 32, 4, 64), (1, 8192, 32, 8, 128)])
def test_flash_at_the_benchmark_shapes(B, T, Hq, Hkv, D):
    """The shapes the training benchmarks run (1.1B: batch 4 x 2048, 32 q / 4 kv heads of 64; 8B: 8192 tokens, 32 q /
    8 kv heads of 128) against fp32 on a subsample of query rows, and dK / dV / dQ against an fp32 reference on one
    (batch, kv head) group."""
    from litetorch_b200.ops import kernels as K
    g = torch.Generator(device="cuda").manual_seed(5)
    q = torch.randn(B, T, Hq, D, device="cuda", generator=g).bfloat16()
    k = torch.randn(B, T, Hkv, D, device="cuda", generator=g).bfloat16()
    v = torch.randn(B, T, Hkv, D, device="cuda", generator=g).bfloat16()
    do = torch.randn(B, T, Hq, D, device="cuda", generator=g).bfloat16()
    scale = D ** -0.5
    o, lse = K.flash_fwd(q, k, v, causal=True, scale=scale)
    dq, dk, dv = K.flash_bwd(q, k, v, o, lse, do, causal=True, scale=scale)
    torch.cuda.synchronize()
    K.check_status()
    rows = torch.cat([torch.arange(0, 130, device="cuda"), torch.randint(0, T, (254,), device="cuda", generator=g),
                      torch.arange(T - 128, T, device="cuda")])
    G = Hq // Hkv
    for b, h in ((0, 0), (B - 1, Hq - 1), (B // 2, Hq // 2 + 1)):
        o_r, lse_r, dq_r = _ref_rows(q[b, :, h], k[b, :, h // G], v[b, :, h // G], do[b, :, h], rows, scale)
        assert _err(o[b, rows, h], o_r) < 1e-2
        assert (lse[b, h, rows] - lse_r).abs().max().item() < 2e-2
        assert _err(dq[b, rows, h], dq_r) < 2e-2
    # dK / dV of one kv head: sum over its G query heads, all rows, in fp32 but one head at a time (T x T fits for one head)
    b, hk = B - 1, Hkv - 1
    dk_r = torch.zeros(T, D, device="cuda")
    dv_r = torch.zeros(T, D, device="cuda")
    kf, vf = k[b, :, hk].float(), v[b, :, hk].float()
    all_rows = torch.arange(T, device="cuda")
    for h in range(hk * G, (hk + 1) * G):
        qf, dof = q[b, :, h].float(), do[b, :, h].float()
        for r0 in range(0, T, 2048):                       # query rows in slabs to bound the score matrix
            rr = all_rows[r0:r0 + 2048]
            s = (qf[rr] @ kf.t() * scale).masked_fill(all_rows[None, :] > rr[:, None], float("-inf"))
            p = torch.softmax(s, -1)
            o_s = p @ vf
            dp = dof[rr] @ vf.t()
            ds = p * (dp - (dof[rr] * o_s).sum(-1, keepdim=True)) * scale
            dv_r += p.t() @ dof[rr]
            dk_r += ds.t() @ qf[rr]
    assert _err(dv[b, :, hk], dv_r) < 2e-2
    assert _err(dk[b, :, hk], dk_r) < 2e-2


@pytest.mark.parametrize("D,H,Hkv,bs", [(64, 32, 4, 16), (64, 8, 8, 8), (64, 16, 1, 32), (128, 32, 8, 16), (128, 12, 3, 64), (64, 6, 2, 16)])
def test_paged_decode_tensor_core_kernel_against_fp32(D, H, Hkv, bs):
    """Decode attention over a paged bf16 cache (tiles by TMA in the swizzled layout, scores and P V on mma.sync): group sizes 1 to 16,
    blocks of 8 to 64 keys, contexts that end inside a block and inside a 32-key chunk, scattered blocks, 1 to 8 context splits."""
    from litetorch_b200.ops import kernels as K
    torch.manual_seed(D + H + bs)
    ctx = [1, 31, 32, 33, 200, 515, 1024, 7]
    S = len(ctx)
    nblk = sum((c + bs - 1) // bs for c in ctx) + 3
    # poisoned cache: slots no context owns hold NaN, as uninitialised memory might
    kc = torch.full((nblk, Hkv, bs, D), float("nan"), device="cuda", dtype=torch.bfloat16)
    vc = torch.full((nblk, Hkv, bs, D), float("nan"), device="cuda", dtype=torch.bfloat16)
    perm = torch.randperm(nblk).tolist()
    maxb = max((c + bs - 1) // bs for c in ctx)
    bt = torch.zeros(S, maxb, dtype=torch.int32)
    ks, vs, used = [], [], 0
    for s_, c in enumerate(ctx):
        nb = (c + bs - 1) // bs
        blocks = perm[used:used + nb]
        used += nb
        bt[s_, :nb] = torch.tensor(blocks)
        k = torch.randn(c, Hkv, D, device="cuda").bfloat16()
        v = torch.randn(c, Hkv, D, device="cuda").bfloat16()
        for t in range(0, c, bs):
            n = min(bs, c - t)
            kc[blocks[t // bs], :, :n] = k[t:t + n].permute(1, 0, 2)
            vc[blocks[t // bs], :, :n] = v[t:t + n].permute(1, 0, 2)
        ks.append(k)
        vs.append(v)
    q = torch.randn(S, H, D, device="cuda").bfloat16()
    cl = torch.tensor(ctx, dtype=torch.int32, device="cuda")
    for splits in (1, 3, 8):
        out = K.paged_decode(q, kc, vc, bt.cuda(), cl, bs, splits, D ** -0.5)
        K.check_status()
        assert torch.isfinite(out.float()).all()
        for s_, c in enumerate(ctx):
            kk = ks[s_].float().permute(1, 0, 2).repeat_interleave(H // Hkv, 0)
            vv = vs[s_].float().permute(1, 0, 2).repeat_interleave(H // Hkv, 0)
            p = torch.softmax(torch.einsum("hd,htd->ht", q[s_].float(), kk) * D ** -0.5, -1)
            ref = torch.einsum("ht,htd->hd", p, vv)
            err = float((out[s_].float() - ref).norm() / ref.norm())
            assert err < 1.5e-2, (s_, c, splits, err)
