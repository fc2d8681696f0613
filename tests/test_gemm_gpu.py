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
