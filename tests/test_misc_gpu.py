"""Router, dropout, softmax, block quantiser, GradScaler step, reductions and strided copy kernels against plain
PyTorch fp32 references."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("N,E,k", [(1000, 8, 2), (513, 64, 6), (300, 256, 8), (7, 3, 1)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_moe_router_forward_backward(N, E, k, dtype):
    from litetorch_b200.ops import functional as Fn
    torch.manual_seed(0)
    logits = (torch.randn(N, E, device="cuda") * 2).to(dtype).requires_grad_(True)
    tw, ti, probs = Fn.moe_router(logits, k, renorm=True)
    ref_l = logits.detach().float().requires_grad_(True)
    p_ref = torch.softmax(ref_l, -1)
    tp, ti_ref = p_ref.topk(k, -1)
    tw_ref = tp / tp.sum(-1, keepdim=True)
    torch.testing.assert_close(probs, p_ref, rtol=1e-4, atol=1e-6)
    # compare as sets per token (ties between equal probabilities may order differently)
    assert torch.equal(ti.sort(-1).values, ti_ref.sort(-1).values)
    torch.testing.assert_close(tw.sort(-1).values, tw_ref.sort(-1).values, rtol=1e-4, atol=1e-6)
    gw = torch.randn(N, k, device="cuda")
    gp = torch.randn(N, E, device="cuda") * 0.1
    # gradient through the weights (gathered in the kernel's order) and through the dense probabilities
    (tw * gw).sum().add((probs * gp).sum()).backward()
    order = ti.argsort(-1)
    order_ref = ti_ref.argsort(-1)
    gw_ref = torch.empty_like(gw)
    gw_ref.scatter_(1, order_ref, gw.gather(1, order))
    (tw_ref * gw_ref).sum().add((p_ref * gp).sum()).backward()
    torch.testing.assert_close(logits.grad.float(), ref_l.grad, rtol=2e-2 if dtype == torch.bfloat16 else 1e-3,
                               atol=2e-3 if dtype == torch.bfloat16 else 1e-5)


def test_router_counts_and_mass():
    from litetorch_b200.ops import kernels as K
    torch.manual_seed(1)
    N, E, k = 4096, 16, 2
    logits = torch.randn(N, E, device="cuda")
    counts = torch.zeros(E, dtype=torch.int32, device="cuda")
    mass = torch.zeros(E, device="cuda")
    probs, tw, ti = K.moe_router(logits, k, counts=counts, mass=mass)
    assert int(counts.sum()) == N * k
    torch.testing.assert_close(counts.long(), torch.bincount(ti.reshape(-1).long(), minlength=E))
    torch.testing.assert_close(mass, probs.sum(0), rtol=1e-4, atol=1e-3)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_dropout_mask_statistics_and_backward(dtype):
    from litetorch_b200.ops import functional as Fn
    torch.manual_seed(3)
    x = torch.ones(1 << 20, device="cuda", dtype=dtype, requires_grad=True)
    p = 0.25
    y = Fn.dropout(x, p, True)
    kept = (y != 0).float().mean().item()
    assert abs(kept - (1 - p)) < 5e-3
    assert torch.allclose(y[y != 0].float(), torch.full_like(y[y != 0], 1 / (1 - p)).float(), rtol=1e-2)
    y.sum().backward()
    assert torch.equal(x.grad != 0, y != 0)          # backward regenerates the same mask
    y2 = Fn.dropout(x.detach(), p, True)
    assert not torch.equal(y2 != 0, y != 0)          # the offset advances between calls
    assert Fn.dropout(x, p, False) is x


@pytest.mark.parametrize("shape", [(64, 1000), (3, 7, 129), (4096, 32), (5, 5000)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_softmax_forward_backward(shape, dtype):
    from litetorch_b200.ops import functional as Fn
    torch.manual_seed(4)
    x = (torch.randn(*shape, device="cuda") * 3).to(dtype).requires_grad_(True)
    y = Fn.softmax(x, -1)
    xr = x.detach().float().requires_grad_(True)
    yr = torch.softmax(xr, -1)
    tol = dict(rtol=2e-2, atol=2e-3) if dtype == torch.bfloat16 else dict(rtol=1e-4, atol=1e-6)
    torch.testing.assert_close(y.float(), yr, **tol)
    g = torch.randn(*shape, device="cuda")
    (y.float() * g).sum().backward()
    (yr * g).sum().backward()
    torch.testing.assert_close(x.grad.float(), xr.grad, **(dict(rtol=5e-2, atol=5e-3) if dtype == torch.bfloat16 else tol))


@pytest.mark.parametrize("N,K", [(256, 512), (300, 1024), (128, 128)])
def test_quant_128x128_matches_reference(N, K):
    from litetorch_b200.ops import kernels as Kn
    torch.manual_seed(5)
    w = (torch.randn(N, K, device="cuda") * 0.05).bfloat16()
    q, sc = Kn.quant_fp8_128x128(w)
    nb = (N + 127) // 128
    wp = torch.nn.functional.pad(w.float(), (0, 0, 0, nb * 128 - N)).view(nb, 128, K // 128, 128)
    sc_ref = wp.abs().amax((1, 3)).clamp_min(1e-12) / 448.0
    torch.testing.assert_close(sc, sc_ref, rtol=1e-6, atol=0)
    deq = (torch.nn.functional.pad(q.float(), (0, 0, 0, nb * 128 - N)).view(nb, 128, K // 128, 128) * sc[:, None, :, None])
    err = (deq - wp).abs().max().item()
    assert err <= wp.abs().max().item() * 0.07


def test_unscale_check_and_grad_scaler():
    from litetorch_b200.ops import kernels as Kn
    g = torch.randn(100003, device="cuda")
    ref = g * 0.125
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    Kn.unscale_check_(g, 0.125, flag)
    torch.testing.assert_close(g, ref)
    assert flag.item() == 0
    g[77] = float("inf")
    Kn.unscale_check_(g, 1.0, flag)
    assert flag.item() == 1
    flag.zero_()
    gb = torch.randn(4096, device="cuda").bfloat16()
    gb[5] = float("nan")
    Kn.unscale_check_(gb, 1.0, flag)
    assert flag.item() == 1


@pytest.mark.parametrize("n", [1, 1000, 1 << 22])
def test_reduce_all(n):
    from litetorch_b200.ops import kernels as Kn
    torch.manual_seed(6)
    x = torch.randn(n, device="cuda")
    torch.testing.assert_close(Kn.reduce_all(x, "sum")[0], x.double().sum().float(), rtol=1e-4, atol=1e-2)
    assert Kn.reduce_all(x, "max")[0].item() == x.max().item()
    xb = x.bfloat16()
    assert Kn.reduce_all(xb, "max")[0].item() == xb.float().max().item()


def test_strided_copy_permute_and_cat():
    from litetorch_b200.ops import kernels as Kn
    torch.manual_seed(7)
    x = torch.randn(6, 5, 4, 3, device="cuda").bfloat16()
    v = x.permute(3, 1, 0, 2)
    out = torch.empty(v.shape, device="cuda", dtype=x.dtype)
    Kn.strided_copy(v, out)
    assert torch.equal(out, v.contiguous())
    a, b = torch.randn(4, 3, device="cuda"), torch.randn(4, 5, device="cuda")
    cat = torch.empty(4, 8, device="cuda")
    Kn.strided_copy(a, cat[:, :3])
    Kn.strided_copy(b, cat[:, 3:])
    assert torch.equal(cat, torch.cat([a, b], 1))


@pytest.mark.parametrize("S,F", [(384, 512), (130, 5632)])
def test_moe_expert_bwd_pointwise(S, F):
    from litetorch_b200.ops import kernels as K
    torch.manual_seed(2)
    gu = torch.randn(S, 2 * F, device="cuda").bfloat16()
    dh_u = torch.randn(S, F, device="cuda").bfloat16()
    w = torch.rand(S, device="cuda")
    slot = torch.stack([torch.randint(0, 4, (S,), device="cuda"), torch.arange(S, device="cuda")], 1).int()
    slot[S // 3::7, 0] = -1                                    # padding slots
    gu[S // 3::7] = float("nan")                                # whatever is there must not leak out
    dgu, hw, dw = K.moe_expert_bwd(gu, dh_u, w, slot.contiguous())
    valid = (slot[:, 0] >= 0)
    g, u = gu[:, :F].float(), gu[:, F:].float()
    sg = torch.sigmoid(g)
    h = (g * sg * u).bfloat16().float()
    dh = (dh_u.float() * w[:, None]).bfloat16().float()
    ref_dg = dh * u * (sg + g * sg * (1 - sg))
    ref_du = dh * g * sg
    ref = torch.cat([ref_dg, ref_du], 1)
    ref_hw = h * w[:, None]
    ref_dw = (h * dh_u.float()).sum(-1)
    z = ~valid
    assert not torch.isnan(dgu.float()).any() and not torch.isnan(hw.float()).any() and not torch.isnan(dw).any()
    assert float(dgu[z].float().abs().max()) == 0 and float(hw[z].float().abs().max()) == 0 and float(dw[z].abs().max()) == 0
    torch.testing.assert_close(dgu[valid].float(), ref[valid], rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(hw[valid].float(), ref_hw[valid], rtol=2e-2, atol=1e-2)
    torch.testing.assert_close(dw[valid], ref_dw[valid], rtol=1e-2, atol=5e-2 * F ** 0.5)


@pytest.mark.parametrize("name", ["SGD", "RMSprop", "AdamW8bit", "AdamWFP8"])
def test_optimizer_kernels_follow_the_torch_path(name):
    """SGD / RMSprop flat kernels and the int8 / e4m3-moment AdamW kernels against the same optimizer's PyTorch path on
    the CPU, over several steps with identical gradients (fp32 reference arithmetic)."""
    import litetorch_b200 as lt
    from litetorch_b200.core import Tensor, _unwrap
    g = torch.Generator().manual_seed(0)
    w0 = torch.randn(257, 33, generator=g)
    grads = [torch.randn(257, 33, generator=g) * (0.5 + k) for k in range(6)]
    kw = {"SGD": dict(lr=0.05, momentum=0.9, weight_decay=0.01), "RMSprop": dict(lr=0.01, alpha=0.95, weight_decay=0.01),
          "AdamW8bit": dict(lr=0.01, weight_decay=0.1), "AdamWFP8": dict(lr=0.01, weight_decay=0.1)}[name]
    res = []
    for dev in ("cpu", "cuda"):
        p = Tensor(w0.clone().to(dev).requires_grad_(True))
        opt = getattr(lt.optim, name)([p], **kw)
        for gr in grads:
            _unwrap(p).grad = gr.to(dev)
            opt.step()
        res.append(_unwrap(p).detach().float().cpu())
        if dev == "cuda" and name.startswith("AdamW"):
            codes = opt.m_q[0] if name == "AdamW8bit" else opt.m8[0]
            assert codes.dtype == (torch.int8 if name == "AdamW8bit" else torch.float8_e4m3fn) and codes.is_cuda
            assert torch.is_tensor(opt.m_scale[0]) and opt.m_scale[0].is_cuda        # scales never left the device
    tol = 1e-5 if name in ("SGD", "RMSprop") else 2e-2      # a code may round the other way when fp32 sums are fused differently
    assert float((res[0] - res[1]).abs().max()) < tol * max(1.0, float(res[0].abs().max()))
