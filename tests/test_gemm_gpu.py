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
