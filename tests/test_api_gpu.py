"""Public API on a B200: bf16 lt.Ops / lt.nn reach the sm_100a kernels; JIT (NVRTC), paged decode, CUDA graphs."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _err(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-9)).item()


def test_functional_ops_use_native_kernels_and_match_torch():
    import litetorch_b200 as lt
    from litetorch_b200.core import _unwrap
    from litetorch_b200.ops import functional as Fn, kernels as K
    torch.manual_seed(0)
    dev = "cuda"
    K.reset_launch_count()
    x = torch.randn(4, 96, 256, device=dev).bfloat16().requires_grad_(True)
    w = (torch.randn(512, 256, device=dev) * 0.05).bfloat16().requires_grad_(True)
    b = torch.randn(512, device=dev).bfloat16().requires_grad_(True)
    y = Fn.linear(x, w, b, act="gelu")
    yr = torch.nn.functional.gelu(x.float() @ w.float().t() + b.float(), approximate="tanh")
    assert _err(y, yr) < 1e-2
    g = torch.randn_like(y)
    y.backward(g)
    gx, gw = torch.autograd.grad(yr, [x, w], g.float())
    assert _err(x.grad, gx) < 2e-2 and _err(w.grad, gw) < 2e-2
    n = torch.ones(256, device=dev).bfloat16().requires_grad_(True)
    r = Fn.rms_norm(x.detach(), n, 1e-5)
    xf = x.detach().float()
    assert _err(r, xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5)) < 1e-2
    a = torch.randn(64, 128, device=dev).bfloat16().requires_grad_(True)
    c = torch.randn(128, 72, device=dev).bfloat16().requires_grad_(True)
    m = Fn.matmul(a, c)
    assert _err(m, a.float() @ c.float()) < 1e-2
    m.sum().backward()
    assert _err(a.grad, torch.ones(64, 72, device=dev) @ c.float().t()) < 1e-2
    q = torch.randn(2, 4, 128, 64, device=dev).bfloat16().requires_grad_(True)
    kk = torch.randn(2, 2, 128, 64, device=dev).bfloat16()
    o = Fn.flash_attention(q, kk, kk, is_causal=True)
    ref = torch.nn.functional.scaled_dot_product_attention(q.float(), kk.float().repeat_interleave(2, 1), kk.float().repeat_interleave(2, 1), is_causal=True)
    assert _err(o, ref) < 1e-2
    o.sum().backward()
    logits = (torch.randn(50, 1000, device=dev) * 2).bfloat16().requires_grad_(True)
    tgt = torch.randint(0, 1000, (50,), device=dev).float()
    loss = Fn.cross_entropy(logits, tgt)
    lr = logits.detach().float().requires_grad_(True)
    ref = torch.nn.functional.cross_entropy(lr, tgt.long())
    assert abs(loss.item() - ref.item()) < 5e-3
    loss.backward()
    ref.backward()
    assert _err(logits.grad, lr.grad) < 2e-2
    assert K.launch_count() >= 12          # the native path ran, not a PyTorch fallback
    K.check_status()
    net = lt.nn.Sequential([lt.nn.Linear(256, 512), lt.nn.GELU(), lt.nn.Linear(512, 256)]).to("cuda:0").cast(lt.BF16)
    out = net(lt.Tensor(x.detach()))
    assert out.shape == [4, 96, 256] and out.dtype == lt.BF16


def test_adam_table_kernel_matches_torch():
    import litetorch_b200 as lt
    from litetorch_b200.core import _unwrap
    torch.manual_seed(0)
    shapes = [(300, 7), (5,), (70000,), (64, 64)]
    ours = [lt.Tensor(torch.randn(*s, device="cuda").requires_grad_(True)) for s in shapes]
    ref = [_unwrap(p).detach().clone().requires_grad_(True) for p in ours]
    oa = lt.optim.AdamW(ours, lr=1e-2, beta1=0.9, beta2=0.95, weight_decay=0.1)
    ob = torch.optim.AdamW(ref, lr=1e-2, betas=(0.9, 0.95), weight_decay=0.1)
    for _ in range(3):
        for p, r in zip(ours, ref):
            g = torch.randn_like(r)
            _unwrap(p).grad = g.clone()
            r.grad = g.clone()
        oa.step()
        ob.step()
    for p, r in zip(ours, ref):
        assert torch.allclose(_unwrap(p), r, atol=1e-5)
    b16 = lt.Tensor(torch.randn(1000, device="cuda").bfloat16().requires_grad_(True))
    o16 = lt.optim.AdamW([b16], lr=1e-2)
    _unwrap(b16).grad = torch.ones(1000, device="cuda").bfloat16()
    before = _unwrap(b16).detach().clone()
    o16.step()
    assert o16.master[0] is not None and o16.master[0].dtype == torch.float32 and not torch.equal(before, _unwrap(b16).detach())


def test_jit_fused_kernel_via_nvrtc():
    import litetorch_b200 as lt
    from litetorch_b200.core import _unwrap
    J = lt.jit
    x, b = J.JITVar.input("x"), J.JITVar.input("b")
    f = J.JITFunction("bias_gelu_res", J.gelu(x + b) * 0.5 + x, [x, b])
    for dt, tol in [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)]:
        a = torch.randn(1000, 64, device="cuda").to(dt).requires_grad_(True)
        c = torch.randn(1000, 64, device="cuda").to(dt)
        out = _unwrap(f(lt.Tensor(a), lt.Tensor(c)))
        ref = torch.nn.functional.gelu(a.float() + c.float(), approximate="tanh") * 0.5 + a.float()
        assert (out.float() - ref).abs().max().item() < tol * 10
        out.sum().backward()
        gr = torch.autograd.grad(ref.sum(), a)[0]
        assert _err(a.grad, gr) < max(tol, 1e-4) * 2
    r = J.fused_bias_relu(lt.Tensor(torch.randn(8, 16, device="cuda")), lt.Tensor(torch.randn(16, device="cuda")))
    assert r.shape == [8, 16] and (_unwrap(r) >= 0).all()


@pytest.mark.parametrize("D,fp8", [(128, False), (64, False), (128, True)])
def test_paged_decode_and_kv_append(D, fp8):
    from litetorch_b200.serving import PagedKVCache, paged_attention
    torch.manual_seed(0)
    S, H, Hkv, bs, nblk = 5, 8, 2, 16, 64
    dtype = torch.float8_e4m3fn if fp8 else torch.bfloat16
    cache = PagedKVCache(1, nblk, bs, Hkv, D, "cuda", dtype, k_scale=0.05 if fp8 else 1.0, v_scale=0.05 if fp8 else 1.0)
    ctx = [37, 200, 1, 64, 129]
    perm = torch.randperm(nblk).tolist()
    maxb = max((c + bs - 1) // bs for c in ctx)
    bt = torch.zeros(S, maxb, dtype=torch.int32)
    ks, vs, used = [], [], 0
    for s, c in enumerate(ctx):
        nb = (c + bs - 1) // bs
        blocks = perm[used:used + nb]
        used += nb
        bt[s, :nb] = torch.tensor(blocks)
        k, v = torch.randn(c, Hkv, D, device="cuda").bfloat16(), torch.randn(c, Hkv, D, device="cuda").bfloat16()
        slots = torch.tensor([blocks[t // bs] * bs + t % bs for t in range(c)], dtype=torch.int32, device="cuda")
        cache.append(0, k, v, slots)
        ks.append(k)
        vs.append(v)
    q = torch.randn(S, H, D, device="cuda").bfloat16()
    cl = torch.tensor(ctx, dtype=torch.int32, device="cuda")
    for splits in (1, 4):
        out = paged_attention(q, cache.k[0], cache.v[0], bt.cuda(), cl, bs, num_splits=splits, k_scale=cache.k_scale, v_scale=cache.v_scale)
        for s, c in enumerate(ctx):
            kk = ks[s].float().permute(1, 0, 2).repeat_interleave(H // Hkv, 0)
            vv = vs[s].float().permute(1, 0, 2).repeat_interleave(H // Hkv, 0)
            p = torch.softmax(torch.einsum("hd,htd->ht", q[s].float(), kk) / math.sqrt(D), -1)
            ref = torch.einsum("ht,htd->hd", p, vv)
            assert _err(out[s], ref) < (0.12 if fp8 else 1.5e-2), (s, splits)


def test_cuda_graph_capture_of_native_kernels_and_compiled_sequential():
    import litetorch_b200 as lt
    from litetorch_b200.core import _unwrap
    from litetorch_b200.cuda import CapturedGraph
    from litetorch_b200.ops import kernels as K
    a = torch.randn(256, 256, device="cuda").bfloat16()
    b = torch.randn(256, 256, device="cuda").bfloat16()
    out = torch.empty(256, 256, device="cuda", dtype=torch.bfloat16)
    K.gemm(a, b, out=out)           # warm-up: function attributes are set outside capture
    g = CapturedGraph()
    with g.capture():
        K.gemm(a, b, out=out)
        K.gelu_fwd(out)
    a.copy_(torch.randn_like(a))
    g.replay()
    torch.cuda.synchronize()
    assert _err(out, a.float() @ b.float().t()) < 1e-2
    net = lt.nn.Sequential([lt.nn.Linear(64, 64), lt.nn.ReLU(), lt.nn.Linear(64, 8)]).to("cuda:0")
    net.compile()
    x = lt.Tensor(torch.randn(16, 64, device="cuda"))
    with torch.no_grad():
        eager = _unwrap(net._run(x)).clone()
        y1 = _unwrap(net(x)).clone()
        x2 = lt.Tensor(torch.randn(16, 64, device="cuda"))
        y2 = _unwrap(net(x2)).clone()
        assert torch.allclose(y1, eager, atol=1e-5) and torch.allclose(y2, _unwrap(net._run(x2)), atol=1e-5)
    assert net._graph is not None


def test_ring_attention_single_rank_uses_flash_kernel_and_zigzag_math():
    import litetorch_b200 as lt
    from litetorch_b200.core import _unwrap
    q = torch.randn(1, 4, 256, 64, device="cuda").bfloat16()
    k = torch.randn(1, 2, 256, 64, device="cuda").bfloat16()
    o = lt.Ops.ring_attention(lt.Tensor(q), lt.Tensor(k), lt.Tensor(k), None, causal=True)
    ref = torch.nn.functional.scaled_dot_product_attention(q.float(), k.float().repeat_interleave(2, 1), k.float().repeat_interleave(2, 1), is_causal=True)
    assert _err(_unwrap(o), ref) < 1e-2
