"""Public API on CPU: Tensor, Ops, nn, optim, amp, quantization (the reference's feature-bundle tests, as pytest)."""
import math

import pytest
import torch

import litetorch_b200 as lt
from litetorch_b200.core import _unwrap


def T(data, shape, grad=False):
    return lt.Tensor.from_vector(data, shape, lt.Device("cpu"), grad)


def test_tensor_basics_and_views():
    x = T([1, 2, 3, 4, 5, 6], [2, 3], True)
    assert x.shape == [2, 3] and x.strides == [3, 1] and x.numel() == 6 and x.dtype == lt.FP32
    assert x.device == lt.Device("cpu") and x.requires_grad
    y = x.transpose(0, 1)
    assert y.shape == [3, 2] and not y.is_contiguous() and y.contiguous().is_contiguous()
    assert x.view([3, 2]).to_vector() == [1, 2, 3, 4, 5, 6]
    c = x.clone()
    c.add_(T([1] * 6, [2, 3]))
    assert c.to_vector()[0] == 2 and x.to_vector()[0] == 1
    z = lt.Tensor.zeros([2, 2])
    z.copy_(T([1, 2, 3, 4], [2, 2]))
    assert z.to_vector() == [1, 2, 3, 4]
    assert lt.Device("cuda:1").index == 1 and lt.Device("cuda:1").type == lt.GPU
    m = lt.Tensor.create([4, 4], lt.Device("meta"))
    assert m.device.type == lt.META and m.shape == [4, 4]


def test_autograd_hooks_and_double_backward():
    x = T([2.0, 3.0], [2], True)
    seen = []
    x.register_hook(lambda g: seen.append(g.to_vector()) or None)
    y = lt.Ops.sum(lt.Ops.mul(lt.Ops.mul(x, x), x))  # sum x^3
    y.backward(create_graph=True)
    assert seen and x.grad.to_vector() == pytest.approx([12.0, 27.0])
    g = _unwrap(x).grad
    x.zero_grad()
    g.sum().backward()  # d/dx sum(3x^2) = 6x
    assert x.grad.to_vector() == pytest.approx([12.0, 18.0])


def test_ops_broadcast_reduce_shape():
    a = T([1, 2, 3, 4, 5, 6], [2, 3], True)
    b = T([10, 20, 30], [3], True)
    c = lt.Ops.add(a, b)
    assert c.to_vector() == [11, 22, 33, 14, 25, 36]
    lt.Ops.sum(c).backward()
    assert b.grad.to_vector() == [2, 2, 2]          # un-broadcast gradient
    assert lt.Ops.mean(a).shape == [1] and lt.Ops.max(a).item() == 6
    assert lt.Ops.cat([a, a], 0).shape == [4, 3]
    assert lt.Ops.unsqueeze(a, 0).shape == [1, 2, 3] and lt.Ops.squeeze(lt.Ops.unsqueeze(a, 0), 0).shape == [2, 3]
    assert lt.Ops.clamp(a, 2, 4).to_vector() == [2, 2, 3, 4, 4, 4]
    for name in ("sqrt", "exp", "log", "abs", "neg", "sin", "cos", "relu", "sigmoid", "tanh", "gelu", "silu"):
        assert getattr(lt.Ops, name)(a).shape == [2, 3]
    assert lt.Ops.softmax(a, -1).to_vector()[:3] == pytest.approx(torch.softmax(torch.tensor([1., 2., 3.]), 0).tolist())
    assert lt.Ops.pow(a, 2.0).to_vector()[2] == 9 and lt.Ops.leaky_relu(lt.Ops.neg(a), 0.1).to_vector()[0] == pytest.approx(-0.1)
    assert lt.Ops.bmm(lt.Tensor.zeros([2, 3, 4]), lt.Tensor.zeros([2, 4, 5])).shape == [2, 3, 5]


def test_matmul_shapes_and_transposed_views():
    a = T(list(range(6)), [2, 3])
    b = T(list(range(12)), [3, 4])
    assert lt.Ops.matmul(a, b).shape == [2, 4]
    w = T(list(range(12)), [4, 3])
    ref = _unwrap(a) @ _unwrap(w).t()
    assert torch.equal(_unwrap(lt.Ops.matmul(a, w.transpose(0, 1))), ref)
    x3 = lt.Tensor.zeros([5, 2, 3])
    assert lt.Ops.matmul(x3, b).shape == [5, 2, 4]
    with pytest.raises(Exception):
        lt.Ops.matmul(a, T([1, 2], [2, 1]))


def test_layers_losses_and_decoder_layer():
    torch.manual_seed(0)
    x = lt.Tensor.from_torch(torch.randn(2, 5, 16))
    ln = lt.nn.LayerNorm([16])
    y = _unwrap(ln(x))
    assert y.mean(-1).abs().max() < 1e-5
    fused = lt.Ops.fused_add_layernorm(x, x, [16], ln.weight, ln.bias)
    assert torch.allclose(_unwrap(fused), torch.nn.functional.layer_norm(_unwrap(x) * 2, (16,)), atol=1e-5)
    rn = lt.nn.RMSNorm(16)
    assert _unwrap(rn(x)).pow(2).mean(-1).sub(1).abs().max() < 1e-3
    mha = lt.nn.MultiHeadAttention(16, 4)
    assert mha(x).shape == [2, 5, 16]
    dec = lt.nn.TransformerDecoderLayer(16, 4, 32)
    out = dec.forward(x)
    assert out.shape == [2, 5, 16]
    lt.Ops.sum(out).backward()
    assert all(p.grad is not None for p in dec.self_attn.parameters())
    logits = T([2.0, 1.0, 0.1, 0.5, 2.5, 0.3], [2, 3], True)
    ce = lt.Ops.cross_entropy_loss(logits, T([0, 1], [2]))
    assert ce.item() == pytest.approx(torch.nn.functional.cross_entropy(_unwrap(logits), torch.tensor([0, 1])).item())
    assert lt.Ops.mse_loss(T([1, 2], [2]), T([1, 4], [2])).item() == pytest.approx(2.0)
    assert lt.Ops.l1_loss(T([1, 2], [2]), T([1, 4], [2])).item() == pytest.approx(1.0)
    assert lt.Ops.bce_loss(T([0.9, 0.1], [2]), T([1, 0], [2])).item() == pytest.approx(-math.log(0.9), rel=1e-4)
    emb = lt.nn.Embedding(10, 4)
    assert emb(T([1, 3, 3], [3])).shape == [3, 4]
    seq = lt.nn.Sequential([lt.nn.Linear(16, 8), lt.nn.GELU(), lt.nn.Dropout(0.0), lt.nn.Linear(8, 2)])
    assert seq(x).shape == [2, 5, 2] and len(seq.parameters()) == 4


def test_module_hooks_train_eval_and_python_subclass():
    class Net(lt.nn.Module):
        def __init__(self):
            super().__init__()
            self.a, self.b = lt.nn.Linear(4, 4), lt.nn.Linear(4, 2)

        def forward(self, x):
            return self.b(lt.Ops.relu(self.a(x)))
    net = Net()
    calls = []
    net.a.register_forward_pre_hook(lambda m, x: calls.append("pre") or None)
    net.a.register_forward_hook(lambda m, x, o: calls.append("post") or None)
    net(lt.Tensor.zeros([3, 4]))
    assert calls == ["pre", "post"] and len(net.parameters()) == 4 and len(net.children()) == 2
    net.eval()
    assert not net.a.training
    net.train()
    assert net.b.training


def test_vision_ops():
    x = lt.Tensor.from_torch(torch.randn(2, 3, 8, 8))
    conv = lt.nn.Conv2d(3, 4, 3, 1, 1)
    y = conv(x)
    assert y.shape == [2, 4, 8, 8]
    assert lt.nn.MaxPool2d(2)(y).shape == [2, 4, 4, 4]
    assert lt.nn.AdaptiveAvgPool2d(1, 1)(y).shape == [2, 4, 1, 1]
    bn = lt.nn.BatchNorm2d(4)
    assert bn(y).shape == [2, 4, 8, 8]
    assert lt.nn.Flatten()(y).shape == [2, 256]
    assert lt.nn.Conv3d(1, 2, 3, 1, 1)(lt.Tensor.zeros([1, 1, 4, 4, 4])).shape == [1, 2, 4, 4, 4]
    assert lt.nn.MaxPool3d(2)(lt.Tensor.zeros([1, 1, 4, 4, 4])).shape == [1, 1, 2, 2, 2]


def test_rope_gqa_attention_and_decoding_paths():
    torch.manual_seed(0)
    B, H, Hkv, Tn, D = 1, 4, 2, 6, 8
    q, k, v = (lt.Tensor.from_torch(torch.randn(B, h, Tn, D)) for h in (H, Hkv, Hkv))
    inv = 1.0 / (10000 ** (torch.arange(0, D, 2).float() / D))
    ang = torch.arange(Tn).float()[:, None] * inv[None]
    cos, sin = lt.Tensor.from_torch(ang.cos()), lt.Tensor.from_torch(ang.sin())
    r = lt.Ops.rope(q, cos, sin)
    assert torch.allclose(_unwrap(r).norm(dim=-1), _unwrap(q).norm(dim=-1), atol=1e-5)      # rotation keeps norms
    assert torch.allclose(_unwrap(r)[:, :, 0], _unwrap(q)[:, :, 0])                          # position 0 unchanged
    o = lt.Ops.flash_attention(q, k, v)
    kk, vv = _unwrap(k).repeat_interleave(2, 1), _unwrap(v).repeat_interleave(2, 1)
    ref = torch.softmax(_unwrap(q) @ kk.transpose(-1, -2) / math.sqrt(D), -1) @ vv
    assert torch.allclose(_unwrap(o), ref, atol=1e-5)
    oc = lt.Ops.flash_attention(q, k, v, is_causal=True)
    assert torch.allclose(_unwrap(oc)[:, :, 0], vv[:, :, 0], atol=1e-5)                      # first token sees itself only
    q1 = lt.Tensor.from_torch(_unwrap(q)[:, :, -1:])
    fd = lt.Ops.flash_decoding(q1, k, v, 3)
    assert torch.allclose(_unwrap(fd), _unwrap(o)[:, :, -1:], atol=1e-5)


def test_paged_attention_matches_dense():
    torch.manual_seed(0)
    S, H, Hkv, D, bs, nblk = 2, 4, 2, 8, 4, 8
    kc, vc = torch.randn(nblk, Hkv, bs, D), torch.randn(nblk, Hkv, bs, D)
    bt = torch.tensor([[3.0, 1.0, 0.0], [5.0, 2.0, 7.0]])
    cl = torch.tensor([6.0, 11.0])
    q = torch.randn(S, H, D)
    out = _unwrap(lt.Ops.paged_attention(lt.Tensor(q), lt.Tensor(kc), lt.Tensor(vc), lt.Tensor(bt), lt.Tensor(cl), bs))
    for s in range(S):
        n = int(cl[s])
        blocks = bt[s].long()[: (n + bs - 1) // bs]
        kk = kc[blocks].permute(1, 0, 2, 3).reshape(Hkv, -1, D)[:, :n].repeat_interleave(2, 0)
        vv = vc[blocks].permute(1, 0, 2, 3).reshape(Hkv, -1, D)[:, :n].repeat_interleave(2, 0)
        ref = torch.softmax(torch.einsum("hd,htd->ht", q[s], kk) / math.sqrt(D), -1)
        assert torch.allclose(out[s], torch.einsum("ht,htd->hd", ref, vv), atol=1e-5)


def test_optimizers_match_torch_and_schedulers():
    torch.manual_seed(0)
    w0 = torch.randn(5, 3)
    for ours, theirs, kw in [
        (lambda p: lt.optim.AdamW(p, lr=1e-2, beta1=0.9, beta2=0.95, weight_decay=0.1),
         lambda p: torch.optim.AdamW(p, lr=1e-2, betas=(0.9, 0.95), weight_decay=0.1), {}),
        (lambda p: lt.optim.Adam(p, lr=1e-2, weight_decay=0.01), lambda p: torch.optim.Adam(p, lr=1e-2, weight_decay=0.01), {}),
        (lambda p: lt.optim.SGD(p, lr=0.1, momentum=0.9, weight_decay=0.01),
         lambda p: torch.optim.SGD(p, lr=0.1, momentum=0.9, weight_decay=0.01), {}),
        (lambda p: lt.optim.RMSprop(p, lr=0.01, alpha=0.9), lambda p: torch.optim.RMSprop(p, lr=0.01, alpha=0.9), {}),
    ]:
        a = lt.Tensor(w0.clone().requires_grad_(True))
        b = w0.clone().requires_grad_(True)
        oa, ob = ours([a]), theirs([b])
        for _ in range(4):
            g = torch.randn(5, 3)
            _unwrap(a).grad = g.clone()
            b.grad = g.clone()
            oa.step()
            ob.step()
        assert torch.allclose(_unwrap(a), b, atol=1e-5), type(oa).__name__
    p = lt.Tensor(w0.clone().requires_grad_(True))
    opt = lt.optim.AdamW([p], lr=1.0)
    sch = lt.optim.CosineAnnealingLR(opt, T_max=10, eta_min=0.1)
    for _ in range(5):
        sch.step()
    assert opt.lr == pytest.approx(0.1 + 0.9 * (1 + math.cos(math.pi * 0.5)) / 2)
    opt.lr = 1.0
    st = lt.optim.StepLR(opt, step_size=2, gamma=0.5)
    for _ in range(4):
        st.step()
    assert opt.lr == pytest.approx(0.25)
    off = lt.optim.AdamW([p], lr=1e-2, offload_to_cpu=True)
    _unwrap(p).grad = torch.ones(5, 3)
    off.step()
    assert off.m[0].device.type == "cpu"


def test_low_bit_optimizers_reduce_state_and_converge():
    torch.manual_seed(0)
    target = torch.randn(64)
    for cls in (lt.optim.AdamW8bit, lt.optim.AdamWFP8):
        p = lt.Tensor(torch.zeros(64, requires_grad=True))
        opt = cls([p], lr=0.05)
        for _ in range(200):
            opt.zero_grad()
            loss = ((_unwrap(p) - target) ** 2).mean()
            loss.backward()
            opt.step()
        assert loss.item() < 0.5 * float((target ** 2).mean()), cls.__name__   # per-tensor linear codes are coarse for v
    o8 = lt.optim.AdamW8bit([p], lr=0.01)
    _unwrap(p).grad = torch.ones(64)
    o8.step()
    assert o8.state_bytes() == 2 * 64           # one byte per element per moment instead of four


def test_grad_scaler_and_autocast():
    p = lt.Tensor(torch.ones(4, requires_grad=True))
    opt = lt.optim.SGD([p], lr=0.1)
    sc = lt.amp.GradScaler(init_scale=4.0, growth_interval=1)
    loss = lt.Ops.sum(lt.Ops.mul(p, p))
    sc.scale(loss).backward()
    assert _unwrap(p).grad[0].item() == pytest.approx(8.0)
    assert sc.step(opt) and _unwrap(p)[0].item() == pytest.approx(0.8)
    sc.update()
    assert sc.get_scale() == 8.0
    _unwrap(p).grad = torch.tensor([float("inf"), 0, 0, 0])
    before = _unwrap(p).clone()
    assert not sc.step(opt)
    sc.update()
    assert sc.get_scale() == 4.0 and torch.equal(_unwrap(p).detach(), before)
    s2 = lt.optim.GradScaler(init_scale=1.0)
    s2._found_inf = True
    s2.update()
    assert s2.scale == 1.0                       # never below 1
    a, b = lt.Tensor(torch.randn(4, 8)), lt.Tensor(torch.randn(8, 4))
    with lt.amp.AutocastGuard(True, lt.BF16):
        assert lt.amp.AutocastGuard.is_enabled()
        assert _unwrap(lt.Ops.matmul(a, b)).dtype == torch.bfloat16
    assert not lt.amp.AutocastGuard.is_enabled()
    assert _unwrap(lt.Ops.matmul(a, b)).dtype == torch.float32


def test_casts_quantization_qat_qlora():
    x = T([0.1, -0.5, 1.0, 3.3, -6.5, 0.0, 0.74, -0.02], [8])
    for dt, tol in [(lt.FP16, 1e-2), (lt.BF16, 5e-2), (lt.FP8_E4M3, 0.3), (lt.FP8_E5M2, 0.6)]:
        back = x.cast(dt).cast(lt.FP32)
        assert back.dtype == lt.FP32 and max(abs(a - b) for a, b in zip(back.to_vector(), x.to_vector())) < tol
    assert x.cast(lt.INT8).to_vector()[3] == 3.0
    nf = lt.Ops.cast(T([0.0, 1.0, -1.0, 0.3], [4]), lt.NF4)
    assert nf.dtype == lt.NF4 and nf.cast(lt.FP32).to_vector()[:3] == pytest.approx([0.0, 1.0, -1.0])
    fp4 = T([0.4, 2.4, -5.0, 6.0], [4]).cast(lt.FP4)
    assert fp4.cast(lt.FP32).to_vector() == pytest.approx([0.5, 2.0, -4.0, 6.0])
    lin = lt.nn.Linear(8, 4)
    w = _unwrap(lin.weight).detach().clone()
    inp = lt.Tensor(torch.randn(3, 8))
    ref = _unwrap(lin(inp)).detach()
    lt.quantization.quantize_linear(lin)
    assert lin.weight.dtype == lt.INT8 and lin.scales.shape == [4]
    assert (_unwrap(lin(inp)) - ref).abs().max() < 0.05
    cal = lt.quantization.Calibrator()
    cal.collect("a", T([-1.0, 3.0], [2]))
    cal.collect("a", T([-2.0, 1.0], [2]))
    assert cal.get_scale("a") == pytest.approx(3.0 / 127) and cal.get_asymmetric_params("a")[0] == pytest.approx(5.0 / 254)
    qat = lt.quantization.QATLinear(lt.nn.Linear(8, 4), 0.01, 0.0, 0.05, 0.0, 8)
    out = qat.forward(inp)
    lt.Ops.sum(out).backward()
    assert qat.weight.grad is not None                                        # straight-through gradient
    fq = lt.Ops.fake_quantize(T([0.123, 5.0], [2]), 0.01, 0.0, 8)
    assert fq.to_vector() == pytest.approx([0.12, 1.27])
    ql = lt.nn.QLoRALinear(8, 4, r=2)
    assert ql(inp).shape == [3, 4] and len(ql.parameters()) == 3
    assert lt.Ops.scaled_matmul(x.cast(lt.FP8_E4M3).view([2, 4]), T([1.0] * 8, [4, 2]).cast(lt.FP8_E4M3), 0.5, 2.0).shape == [2, 2]
    w8 = lt.Ops.w8a8_matmul(lt.Tensor(torch.randn(4, 8)), lt.Tensor(torch.randn(6, 8)), 0.02, 0.02)      # w is [N, K]
    assert w8.shape == [4, 6]


def test_moe_layer_grads_and_gate():
    torch.manual_seed(0)
    moe = lt.nn.MoELinear(8, 6, 4, 2)
    x = lt.Tensor(torch.randn(10, 8, requires_grad=True))
    y = moe(x)
    assert y.shape == [10, 6]
    lt.Ops.sum(y).backward()
    assert moe.gate_weight.grad is not None and sum(e.weight.grad is not None for e in moe.experts) >= 2
    probs, idx = lt.Ops.moe_gate(x, moe.gate_weight, 2)
    assert probs.shape == [10, 2] and torch.allclose(_unwrap(probs).sum(-1), torch.ones(10))
    assert _unwrap(idx).dtype == torch.float32


def test_fused_linear_cross_entropy_and_clip_and_checkpoint():
    torch.manual_seed(0)
    x = lt.Tensor(torch.randn(10, 8, requires_grad=True))
    w = lt.Tensor(torch.randn(16, 8, requires_grad=True))
    t = T([float(i % 16) for i in range(10)], [10])
    loss = lt.Ops.fused_linear_cross_entropy(x, w, t, chunk_rows=4)
    ref = torch.nn.functional.cross_entropy(_unwrap(x) @ _unwrap(w).t(), _unwrap(t).long())
    assert loss.item() == pytest.approx(ref.item(), rel=1e-5)
    loss.backward()
    g = torch.autograd.grad(ref, _unwrap(w))[0]
    assert torch.allclose(_unwrap(w).grad, g, atol=1e-5)
    n = lt.Ops.clip_grad_norm_([x, w], 0.1)
    assert n > 0.1 and math.sqrt(sum(float(_unwrap(p).grad.pow(2).sum()) for p in (x, w))) == pytest.approx(0.1, rel=1e-3)
    lin = lt.nn.Linear(8, 8)
    xin = lt.Tensor(torch.randn(2, 8, requires_grad=True))
    a = lt.checkpoint(lambda z: lt.Ops.gelu(lin(z)), xin)
    lt.Ops.sum(a).backward()
    g1 = _unwrap(xin).grad.clone()
    xin.zero_grad()
    lt.Ops.sum(lt.Ops.gelu(lin(xin))).backward()
    assert torch.allclose(g1, _unwrap(xin).grad)
    assert lt.Ops.checkpoint(lin, xin).shape == [2, 8]


def test_gpt_config_trains_on_cpu():
    from litetorch_b200.models.gpt import train
    out = train(steps=6, verbose=False)
    assert abs(out["losses"][0] - math.log(256)) < 0.1 and out["tokens_per_s"] > 0


def test_custom_op_registry():
    lt.custom_ops.Registry.register(
        "cube", lambda x: lt.Tensor(_unwrap(x) ** 3),
        backward=lambda inputs, out, g: [lt.Tensor(3 * _unwrap(inputs[0]) ** 2 * _unwrap(g))])
    x = T([1.0, 2.0], [2], True)
    y = lt.custom_ops.Registry.call("cube", [x])
    lt.Ops.sum(y).backward()
    assert y.to_vector() == [1.0, 8.0] and x.grad.to_vector() == [3.0, 12.0]
    assert lt.custom_ops.Registry.has("cube")
    with pytest.raises(KeyError):
        lt.custom_ops.Registry.call("nope", [x])


def test_functional_fallbacks_softmax_dropout_router_fp8_linear():
    """CPU paths of the ops whose CUDA versions are hand-written kernels."""
    import torch
    from litetorch_b200.ops import functional as Fn
    torch.manual_seed(0)
    x = torch.randn(4, 7, 33, requires_grad=True)
    y = Fn.softmax(x, -1)
    torch.testing.assert_close(y, torch.softmax(x, -1))
    y.sum().backward()
    assert x.grad.abs().max() < 1e-6          # d(sum softmax)/dx = 0
    d = Fn.dropout(torch.ones(10000), 0.3, True)
    assert abs(float((d != 0).float().mean()) - 0.7) < 0.03
    assert Fn.dropout(x, 0.3, False) is x
    logits = torch.randn(64, 8, requires_grad=True)
    tw, ti, probs = Fn.moe_router(logits, 2, renorm=True)
    assert ti.shape == (64, 2) and torch.allclose(tw.sum(-1), torch.ones(64), atol=1e-6)
    torch.testing.assert_close(probs.sum(-1), torch.ones(64))
    (tw * torch.randn(64, 2)).sum().backward()
    assert logits.grad is not None and torch.isfinite(logits.grad).all()
    a, w = torch.randn(8, 256), torch.randn(128, 256)
    torch.testing.assert_close(Fn.linear_fp8(a, w), a @ w.t())      # falls back to the plain linear off the GPU
    q = torch.randn(2, 16, 4, 32)
    cos = torch.cos(torch.arange(16)[:, None] * torch.ones(16)[None, :] * 0.1)
    sin = torch.sin(torch.arange(16)[:, None] * torch.ones(16)[None, :] * 0.1)
    torch.testing.assert_close(Fn.rope_bthd(q, cos, sin), Fn.rope(q.transpose(1, 2), cos, sin).transpose(1, 2))


def test_moe_capacity_positions_and_section_timer():
    """The router's capacity cut keeps, per expert, the first `cap` slots in token order (the sort-based position equals
    a running count per expert), and the section timer is inert without a GPU."""
    import math
    from litetorch_b200.parallel.ep import MoEFeedForward
    from litetorch_b200.utils import sections
    torch.manual_seed(4)
    moe = MoEFeedForward(16, 32, 4, top_k=2, capacity_factor=0.6, device="cpu", dtype=torch.float32)
    x = torch.randn(50, 16)
    top_w, top_i, keep, aux = moe.route(x)
    cap = max(1, int(math.ceil(0.6 * 50 * 2 / 4)))
    seen = [0, 0, 0, 0]
    ref = torch.zeros_like(keep)
    for n in range(50):
        for j in range(2):
            e = int(top_i[n, j])
            ref[n, j] = seen[e] < cap
            seen[e] += 1
    assert torch.equal(keep, ref) and not bool(keep.all()) and float(aux) > 0
    with sections.section("x"):
        pass
    assert sections.report() == {} or not torch.cuda.is_available()


def test_run_config_presets_json_and_env(tmp_path):
    from litetorch_b200 import config as C
    assert set(C.PRESETS) == {"gpt-cpu", "llama-1.1b-fsdp", "llama3-8b-fsdp-tp2", "llama3-8b-tp8", "llama3-8b-tp8-fp8",
                              "moe-8x2b-ep8", "llama-3b-long-hybrid"}
    hy = C.load("llama-3b-long-hybrid", env={})
    assert hy.mesh_sizes(8) == {"dp": 1, "tp": 2, "pp": 2, "cp": 2, "ep": 1} and hy.tokens_per_step(8) == 8 * 32768
    assert C.load("llama-1.1b-fsdp", env={}).tokens_per_step(8) == 8 * 4 * 2048
    assert C.load("llama3-8b-tp8-fp8", env={}).precision == "fp8"
    with pytest.raises(ValueError):
        hy.mesh_sizes(4)
    # JSON round trip, unknown fields refused
    path = str(tmp_path / "job.json")
    hy.to_json(path)
    again = C.load(path, env={})
    assert again.to_dict() == hy.to_dict()
    with pytest.raises(KeyError):
        C.RunConfig.from_dict({"model": {"n_layer": 3}})
    # environment overrides: top-level field and SECTION__FIELD, typed by the field's default
    env = {"LT_CFG_SEQ_LEN": "4096", "LT_CFG_PARALLEL__TP": "4", "LT_CFG_ACTIVATION_CHECKPOINTING": "true",
           "LT_CFG_OPTIM__LR": "1e-4", "UNRELATED": "x"}
    c = C.load("llama-1.1b-fsdp", env=env)
    assert c.seq_len == 4096 and c.parallel.tp == 4 and c.activation_checkpointing is True and c.optim.lr == 1e-4
    with pytest.raises(KeyError):
        C.load("llama-1.1b-fsdp", env={"LT_CFG_PARALLEL__NOPE": "1"})
    d = c.decoder_config()
    assert (d.n_layers, d.d_model, d.n_q, d.n_kv) == (22, 2048, 32, 4)
    assert C.load("llama-1.1b-fsdp", env={}).llama_config().num_params() > 1.0e9


def test_logger_and_metrics_writer(tmp_path):
    import io
    import json as _json
    from litetorch_b200.utils.logging import MetricsWriter, get_logger
    buf = io.StringIO()
    log = get_logger("lt-test", level="WARNING", stream=buf)
    log.info("hidden")
    log.warning("shown %d", 7)
    out = buf.getvalue()
    assert "hidden" not in out and "shown 7" in out and out.startswith("[rank 0]")
    path = str(tmp_path / "m.jsonl")
    with MetricsWriter(path) as mw:
        mw.write(step=1, loss=2.5, tokens_per_s=1000.0)
        mw.write(step=2, loss=2.25, tokens_per_s=1100.0, exposed_comm_ms=0.5)
    recs = [_json.loads(l) for l in open(path)]
    assert [r["step"] for r in recs] == [1, 2] and recs[1]["exposed_comm_ms"] == 0.5 and recs[0]["rank"] == 0


def test_vit_trains_on_synthetic_images():
    from litetorch_b200.models.vit import ViT, ViTConfig, synthetic_images, train
    cfg = ViTConfig()
    model = ViT(cfg)
    x, y = synthetic_images(8, cfg)
    logits = model(lt.Tensor(x))
    assert logits.shape == [8, 2]
    lt.Ops.cross_entropy_loss(logits, lt.Tensor(y)).backward()
    assert all(p.grad is not None for p in model.parameters())
    assert any(p is model.pos for p in model.parameters())
    out = train(epochs=3, images=128, verbose=False)
    assert out["loss"][-1] < 0.5 * out["loss"][0] and out["accuracy"][-1] > 0.9 and out["inference_ms_per_image"] > 0
