"""tcgen05 GEMM against an fp32 PyTorch reference: all operand layouts, tails, epilogues."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(a, b, a_major, b_major):
    A = a.float() if a_major == 0 else a.float().t()
    B = b.float().t() if b_major == 0 else b.float()
    return A @ B


def _rel_err(out, ref):
    return ((out.float() - ref).norm() / (ref.norm() + 1e-6)).item()


@pytest.mark.parametrize("a_major,b_major", [(0, 0), (0, 1), (1, 1), (1, 0)])
@pytest.mark.parametrize("M,N,K", [(256, 512, 256), (128, 256, 64), (384, 640, 448), (200, 264, 136), (1024, 2048, 1024)])
@pytest.mark.parametrize("block_n", [128, 256])
def test_gemm_layouts(a_major, b_major, M, N, K, block_n):
    from litetorch_b200.ops import kernels as K_
    torch.manual_seed(0)
    dev = "cuda"
    a = torch.randn((M, K) if a_major == 0 else (K, M), device=dev).bfloat16()
    b = torch.randn((N, K) if b_major == 0 else (K, N), device=dev).bfloat16()
    out = K_.gemm(a, b, a_major=a_major, b_major=b_major, block_n=block_n)
    torch.cuda.synchronize()
    K_.check_status()
    ref = _ref(a, b, a_major, b_major)
    assert _rel_err(out, ref) < 1e-2


def test_gemm_epilogues():
    from litetorch_b200.ops import kernels as K_
    torch.manual_seed(1)
    M, N, K = 512, 768, 320
    a = torch.randn(M, K, device="cuda").bfloat16()
    b = (torch.randn(N, K, device="cuda") * 0.05).bfloat16()
    bias = torch.randn(N, device="cuda").bfloat16()
    res = torch.randn(M, N, device="cuda").bfloat16()
    ref = a.float() @ b.float().t()
    out = K_.gemm(a, b, bias=bias)
    assert _rel_err(out, ref + bias.float()) < 1e-2
    out = K_.gemm(a, b, bias=bias, act=1)
    assert _rel_err(out, torch.nn.functional.gelu(ref + bias.float(), approximate="tanh")) < 1e-2
    out = K_.gemm(a, b, residual=res)
    assert _rel_err(out, ref + res.float()) < 1e-2
    acc = torch.randn(M, N, device="cuda")
    acc0 = acc.clone()
    K_.gemm(a, b, out=acc, accumulate=True, alpha=0.5)
    assert _rel_err(acc, acc0 + 0.5 * ref) < 1e-2
    out32 = K_.gemm(a, b, out_dtype=torch.float32)
    assert _rel_err(out32, ref) < 1e-3
    K_.check_status()


def test_gemm_strided_rows():
    from litetorch_b200.ops import kernels as K_
    torch.manual_seed(2)
    big = torch.randn(300, 1024, device="cuda").bfloat16()
    a = big[:, 128:128 + 256]
    b = torch.randn(192, 256, device="cuda").bfloat16()
    out = K_.gemm(a, b)
    assert _rel_err(out, a.float() @ b.float().t()) < 1e-2
    K_.check_status()


@pytest.mark.parametrize("M,N,K,a_major,b_major,block_n", [
    (8192, 2048, 2048, 0, 0, 256),    # 512 tiles on 148 SMs: the last wave is cut in two
    (2560, 2048, 8192, 1, 1, 256),    # weight-gradient shape: 160 tiles, 12 of them cut eight ways
    (4096, 2560, 512, 0, 1, 128),     # 128-wide tiles, short K
    (8192, 2560, 2048, 0, 0, 0),      # tile width chosen by the cost model
])
@pytest.mark.parametrize("pair_mode", [0, 2])
def test_gemm_split_tail(M, N, K, a_major, b_major, block_n, pair_mode):
    """The K-split of the last tile wave gives the same result as whole tiles, call after call."""
    from litetorch_b200.ops import kernels as K_
    K_.gemm_set_pair_mode(pair_mode)
    torch.manual_seed(1)
    dev = "cuda"
    a = (torch.randn((M, K) if a_major == 0 else (K, M), device=dev) * 0.5).bfloat16()
    b = (torch.randn((N, K) if b_major == 0 else (K, N), device=dev) * 0.5).bfloat16()
    bias = torch.randn(N, device=dev).bfloat16()
    ref = _ref(a, b, a_major, b_major) + bias.float()
    try:
        K_.gemm_set_tail_split(False)
        whole = K_.gemm(a, b, a_major=a_major, b_major=b_major, block_n=block_n, bias=bias)
        K_.gemm_set_tail_split(True)
        outs = [K_.gemm(a, b, a_major=a_major, b_major=b_major, block_n=block_n, bias=bias) for _ in range(3)]
    finally:
        K_.gemm_set_tail_split(True)
    torch.cuda.synchronize()
    K_.check_status()
    K_.gemm_set_pair_mode(1)
    for o in outs:
        assert _rel_err(o, ref) < 1e-2
        # fp32 partial sums are added in a different order: bf16 results may differ in the last place only
        assert (o.float() - whole.float()).abs().max().item() <= 0.02 * ref.abs().max().item()
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[1], outs[2])
    acc = torch.ones(M, N, device=dev, dtype=torch.float32)
    K_.gemm(a, b, a_major=a_major, b_major=b_major, block_n=block_n, out=acc, accumulate=True)
    torch.cuda.synchronize()
    K_.check_status()
    assert _rel_err(acc, _ref(a, b, a_major, b_major) + 1.0) < 1e-2


@pytest.mark.parametrize("a_major,b_major", [(0, 0), (0, 1), (1, 1), (1, 0)])
@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (512, 768, 448), (200, 264, 136), (1000, 520, 256), (4096, 2048, 1024)])
def test_gemm_cta_pairs(a_major, b_major, M, N, K):
    """The cta_group::2 kernel (256 x 256 tiles on CTA pairs) against the fp32 reference, tails included."""
    from litetorch_b200.ops import kernels as K_
    torch.manual_seed(2)
    dev = "cuda"
    a = torch.randn((M, K) if a_major == 0 else (K, M), device=dev).bfloat16()
    b = torch.randn((N, K) if b_major == 0 else (K, N), device=dev).bfloat16()
    bias = torch.randn(N, device=dev).bfloat16()
    res = torch.randn(M, N, device=dev).bfloat16()
    try:
        K_.gemm_set_pair_mode(2)
        out = K_.gemm(a, b, a_major=a_major, b_major=b_major, bias=bias, residual=res)
        out2 = K_.gemm(a, b, a_major=a_major, b_major=b_major, out_dtype=torch.float32)
    finally:
        K_.gemm_set_pair_mode(1)
    torch.cuda.synchronize()
    K_.check_status()
    ref = _ref(a, b, a_major, b_major)
    assert _rel_err(out2, ref) < 1e-2
    assert _rel_err(out, ref + bias.float() + res.float()) < 1e-2


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
@pytest.mark.parametrize("M,N,K", [(256, 384, 512), (1000, 264, 136), (8, 8, 8)])
def test_gemm_fp16_and_tf32_all_layouts(dtype, M, N, K):
    """fp16 (kind::f16) and fp32-as-tf32 (kind::tf32) operands through the same tcgen05 kernels, three operand layouts,
    against fp64 PyTorch; tf32 keeps 10 mantissa bits, so its bound is looser."""
    from litetorch_b200.ops import kernels as KK
    g = torch.Generator(device="cuda").manual_seed(0)
    a = torch.randn(M, K, device="cuda", generator=g).to(dtype)
    b = torch.randn(N, K, device="cuda", generator=g).to(dtype)
    tol = 2e-3
    ref = (a.double() @ b.double().t())
    def err(x, r):
        return float((x.double() - r).norm() / r.norm())
    assert err(KK.gemm_any(a, b), ref) < tol                                                     # x @ W^T
    assert err(KK.gemm_any(a, b.t().contiguous(), b_major=1), ref) < tol                         # A @ B
    assert err(KK.gemm_any(a.t().contiguous(), b.t().contiguous(), a_major=1, b_major=1), ref) < tol   # A^T @ B
    KK.check_status()


def test_linear_matmul_bmm_ops_reach_the_tensor_cores_for_fp32_and_fp16():
    import litetorch_b200 as lt
    from litetorch_b200.core import Tensor, _unwrap
    from litetorch_b200.ops import kernels as K
    g = torch.Generator(device="cuda").manual_seed(1)
    for dtype in (torch.float32, torch.float16, torch.bfloat16):
        x = torch.randn(4, 64, 128, device="cuda", generator=g).to(dtype).requires_grad_(True)
        w = (torch.randn(96, 128, device="cuda", generator=g) * 0.1).to(dtype).requires_grad_(True)
        n0 = K.launch_count()
        y = _unwrap(lt.Ops.bmm(Tensor(x), Tensor(w.t().contiguous().expand(4, 128, 96).contiguous())))
        assert K.launch_count() > n0                          # our GEMM ran (not a library fallback)
        ref = x.detach().double() @ w.detach().double().t()
        assert float((y.double() - ref).norm() / ref.norm()) < 1e-2
        lin = lt.nn.Linear(128, 96)
        lin.to(lt.Device("cuda")) if hasattr(lt, "Device") else None
    # autograd through the fp32 (tf32) linear
    from litetorch_b200.ops import functional as Fn
    x = torch.randn(256, 128, device="cuda", generator=g, requires_grad=True)
    w = (torch.randn(96, 128, device="cuda", generator=g) * 0.1).requires_grad_(True)
    b = torch.randn(96, device="cuda", generator=g, requires_grad=True)
    n0 = K.launch_count()
    y = Fn.linear(x, w, b)
    y.square().sum().backward()
    assert K.launch_count() >= n0 + 3
    xr, wr, br = (t.detach().double().requires_grad_(True) for t in (x, w, b))
    (torch.nn.functional.linear(xr, wr, br)).square().sum().backward()
    for got, want in ((x.grad, xr.grad), (w.grad, wr.grad), (b.grad, br.grad)):
        assert float((got.double() - want).norm() / want.norm()) < 5e-3


@pytest.mark.parametrize("M,N,K", [(1, 2048, 2048), (3, 1000, 264), (8, 11264, 2048), (5, 2048, 5632)])
def test_weight_streaming_gemm_for_a_few_rows(M, N, K):
    """`gemm` with at most eight rows takes the warp-per-column kernel; result (with and without a fused residual)
    against fp32 PyTorch."""
    from litetorch_b200.ops import kernels as KK
    g = torch.Generator(device="cuda").manual_seed(2)
    x = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.05).bfloat16()
    r = torch.randn(M, N, device="cuda", generator=g).bfloat16()
    ref = x.float() @ w.float().t()
    y = KK.gemm(x, w)
    assert float((y.float() - ref).abs().max() / ref.abs().max()) < 1e-2
    y2 = KK.gemm(x, w, residual=r)
    ref2 = ref + r.float()
    assert float((y2.float() - ref2).abs().max() / ref2.abs().max()) < 1e-2
    KK.check_status()


def test_int8_gemm_and_quantisers_are_exact():
    """tcgen05 kind::i8: integer sums are exact, so the result must equal an int64 reference bit for bit; the per-tensor and
    per-row quantisers against the PyTorch formulas; `Ops.w8a8_matmul` through them."""
    import litetorch_b200 as lt
    from litetorch_b200.core import Tensor, _unwrap
    from litetorch_b200.ops import kernels as KK
    g = torch.Generator(device="cuda").manual_seed(3)
    for (M, N, Kd) in [(256, 384, 512), (100, 72, 48), (1000, 264, 2048)]:
        a = torch.randint(-127, 128, (M, Kd), device="cuda", generator=g, dtype=torch.int8)
        b = torch.randint(-127, 128, (N, Kd), device="cuda", generator=g, dtype=torch.int8)
        c = KK.gemm_i8(a, b, alpha=0.5)
        ref = (a.double() @ b.double().t()) * 0.5          # exact: every partial sum is an integer below 2^53
        assert torch.equal(c.double(), ref), (M, N, Kd)
    x = torch.randn(300, 160, device="cuda", generator=g)
    q = KK.quant_int8_tensor(x, 0.03)
    assert torch.equal(q, torch.clamp(torch.round(x / 0.03), -127, 127).to(torch.int8))
    qr, sc = KK.quant_int8_rows(x.bfloat16())
    xb = x.bfloat16().float()
    sref = xb.abs().amax(1) / 127.0
    assert float((sc - sref).abs().max()) < 1e-6
    assert int((qr.int() - torch.clamp(torch.round(xb / sref[:, None]), -127, 127).int()).abs().max()) <= 1
    w = torch.randn(96, 160, device="cuda", generator=g)                   # [N, K], one row per output feature
    y = _unwrap(lt.Ops.w8a8_matmul(Tensor(x), Tensor(w), 0.03, 0.02))
    yr = torch.clamp(torch.round(x / 0.03), -127, 127) @ torch.clamp(torch.round(w / 0.02), -127, 127).t() * (0.03 * 0.02)
    assert y.shape == (300, 96)
    assert float((y - yr).abs().max()) < 1e-3
    KK.check_status()


@pytest.mark.parametrize("M", [9, 16, 17, 32, 33, 64, 100, 128])
@pytest.mark.parametrize("N,Kd", [(2048, 2048), (2560, 2048), (11264, 2048), (2048, 5632), (1000, 64), (32000, 2048), (40, 4096)])
def test_skinny_gemm_against_fp32(M, N, Kd):
    """9 to 128 rows go to the weight-streaming mma.sync kernel (K split over the warps of a CTA and, for narrow outputs, over
    CTAs whose partial sums the last one adds in a fixed order): against fp32, with and without a residual, twice for bit equality."""
    from litetorch_b200.ops import kernels as KK
    torch.manual_seed(M + N)
    a = torch.randn(M, Kd, device="cuda").bfloat16()
    b = (torch.randn(N, Kd, device="cuda") * 0.05).bfloat16()
    res = torch.randn(M, N, device="cuda").bfloat16()
    ref = a.float() @ b.float().t()
    y = KK.gemm(a, b)
    y2 = KK.gemm(a, b)
    KK.check_status()
    assert y.shape == (M, N) and torch.equal(y, y2)
    assert float((y.float() - ref).norm() / ref.norm()) < 6e-3
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    KK.gemm(a, b, out=out, residual=res)
    assert float((out.float() - (ref + res.float())).norm() / (ref + res.float()).norm()) < 6e-3
    # the same product with K split over several CTAs per column group (off by default for short K)
    KK.gemm_skinny_set_target(4, 1)
    try:
        ys = KK.gemm(a, b)
        ys2 = KK.gemm(a, b)
    finally:
        KK.gemm_skinny_set_target()
    assert torch.equal(ys, ys2) and float((ys.float() - ref).norm() / ref.norm()) < 6e-3
    # rows of a wider buffer (strided operands)
    wide = torch.randn(M, Kd + 64, device="cuda").bfloat16()
    y3 = KK.gemm(wide[:, :Kd], b)
    assert float((y3.float() - wide[:, :Kd].float() @ b.float().t()).norm() / ref.norm()) < 6e-3
