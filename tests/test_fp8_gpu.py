"""Block-scaled fp8 GEMM (tcgen05 kind::f8f6f4 with two-level accumulation) against a plain fp32 reference of the
same quantised operands, and the fused 1x128 quantiser against the PyTorch one."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _dequant_a(q, st):
    M, K = q.shape
    return (q.float().view(M, K // 128, 128) * st.t().contiguous()[..., None]).view(M, K)


def _dequant_b(q, s):
    N, K = q.shape
    nb = (N + 127) // 128
    pad = nb * 128 - N
    qf = torch.nn.functional.pad(q.float(), (0, 0, 0, pad))
    d = (qf.view(nb, 128, K // 128, 128) * s[:, None, :, None]).view(nb * 128, K)
    return d[:N]


@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (256, 384, 512), (1000, 520, 1024), (4096, 2048, 2048)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("pairs", [False, True])
def test_fp8_block_gemm_matches_fp32_reference(M, N, K, out_dtype, pairs):
    from litetorch_b200.ops import kernels as Kn
    torch.manual_seed(0)
    dev = "cuda"
    x = (torch.randn(M, K, device=dev) * torch.rand(M, 1, device=dev) * 3).bfloat16()
    w = torch.randn(N, K, device=dev) * 0.05
    xq, xst = Kn.quant_fp8_1x128(x)
    nb = (N + 127) // 128
    wp = torch.nn.functional.pad(w, (0, 0, 0, nb * 128 - N))
    wb = wp.view(nb, 128, K // 128, 128)
    ws = (wb.abs().amax((1, 3)).clamp_min(1e-12) / 448.0).contiguous()
    wq = (wb / ws[:, None, :, None]).clamp(-448, 448).to(torch.float8_e4m3fn).view(nb * 128, K)[:N].contiguous()
    bias = torch.randn(N, device=dev).bfloat16()
    out = Kn.gemm_fp8_block(xq, xst, wq, ws, bias=bias, out_dtype=out_dtype, pairs=pairs)
    ref = _dequant_a(xq, xst) @ _dequant_b(wq, ws).t() + bias.float()
    tol = 2e-2 if out_dtype == torch.bfloat16 else 2e-4
    err = (out.float() - ref).abs().max().item() / ref.abs().max().item()
    assert err < tol, err
    assert Kn.status_fetch() == 0


def test_quant_1x128_matches_torch():
    from litetorch_b200.ops import kernels as Kn
    from litetorch_b200.quantization import quantize_fp8_1x128
    torch.manual_seed(1)
    x = (torch.randn(300, 512, device="cuda") * 2).bfloat16()
    q, st = Kn.quant_fp8_1x128(x)
    q_ref, s_ref = quantize_fp8_1x128(x)
    torch.testing.assert_close(st.t().contiguous(), s_ref, rtol=1e-6, atol=0)
    diff = (q.float() - q_ref.float()).abs()
    # the two roundings may differ by one code where x / scale falls on a tie after the reciprocal multiply
    assert (diff > 0).float().mean().item() < 1e-2
    assert (_dequant_a(q, st) - x.float()).abs().max().item() <= x.float().abs().max().item() * 0.07


def test_fp8_block_linear_close_to_bf16():
    from litetorch_b200.quantization import fp8_block_linear
    torch.manual_seed(2)
    x = torch.randn(512, 1024, device="cuda").bfloat16()
    w = (torch.randn(768, 1024, device="cuda") * 0.03).bfloat16()
    y = fp8_block_linear(x, w)
    ref = x.float() @ w.float().t()
    rel = (y.float() - ref).norm() / ref.norm()
    assert rel < 0.05, rel


@pytest.mark.parametrize("scaling", ["rows", "block"])
def test_linear_fp8_autograd_close_to_bf16(scaling):
    from litetorch_b200.ops import functional as Fn
    torch.manual_seed(3)
    x = torch.randn(512, 1024, device="cuda").bfloat16().requires_grad_(True)
    w = (torch.randn(768, 1024, device="cuda") * 0.03).bfloat16().requires_grad_(True)
    y = Fn.linear_fp8(x, w, scaling=scaling)
    g = torch.randn_like(y)
    y.backward(g)
    xr, wr = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    yr = xr @ wr.t()
    yr.backward(g.float())
    rel = lambda a, b: ((a.float() - b).norm() / b.norm()).item()   # noqa: E731
    assert rel(y, yr) < 0.05
    assert rel(x.grad, xr.grad) < 0.06
    assert rel(w.grad, wr.grad) < 0.02


@pytest.mark.parametrize("M,N,Kd", [(256, 256, 256), (8192, 2816, 2048), (300, 520, 4096), (1000, 136, 48), (129, 4096, 14336)])
def test_gemm_e4m3_row_scaled_is_exact_on_the_codes(M, N, Kd):
    """The row-scaled e4m3 GEMM (tcgen05 kind::f8f6f4, whole K in tensor memory, scales in the epilogue) against the same product
    of the dequantised codes in float64: the only error left is the fp32 accumulation and the rounding of the output."""
    from litetorch_b200.ops import kernels as K
    torch.manual_seed(M + N + Kd)
    x = torch.randn(M, Kd, device="cuda").bfloat16()
    x[:, ::7] *= 8                                           # rows with a wide dynamic range
    w = (torch.randn(N, Kd, device="cuda") * 0.05).bfloat16()
    xq, xs = K.quant_e4m3_rows(x)
    wq, ws = K.quant_e4m3_rows(w)
    assert float((xq.float() * xs[:, None] - x.float()).abs().max() / x.float().abs().max()) < 0.07   # e4m3: 3 mantissa bits
    assert float(xq.float().abs().max()) <= 448.0
    ref = (xq.double() * xs[:, None].double()) @ (wq.double() * ws[:, None].double()).t()
    y32 = K.gemm_e4m3(xq, xs, wq, ws, out_dtype=torch.float32)
    K.check_status()
    acc_err = float((y32.double() - ref).norm() / ref.norm())
    assert acc_err < 1e-3, acc_err
    res = torch.randn(M, N, device="cuda").bfloat16()
    bias = torch.randn(N, device="cuda").bfloat16()
    y16 = K.gemm_e4m3(xq, xs, wq, ws, bias=bias, residual=res)
    full = ref + bias.double()[None] + res.double()
    assert float((y16.double() - full).norm() / full.norm()) < 6e-3
    # against the unquantised product: the quantisation error itself
    exact = x.double() @ w.double().t()
    assert float((y32.double() - exact).norm() / exact.norm()) < 0.06
    assert torch.equal(K.gemm_e4m3(xq, xs, wq, ws, out_dtype=torch.float32), y32)


def test_scaled_matmul_runs_e4m3_codes_on_the_tensor_cores():
    """lt.Ops.scaled_matmul on two e4m3 tensors with per-tensor scales: the tcgen05 kind::f8f6f4 GEMM against float64 on the codes."""
    import litetorch_b200 as lt
    from litetorch_b200.core import _unwrap
    from litetorch_b200.ops import kernels as K
    torch.manual_seed(11)
    a = (torch.randn(200, 96, device="cuda") * 3).to(torch.float8_e4m3fn)
    b = (torch.randn(96, 72, device="cuda") * 3).to(torch.float8_e4m3fn)       # [K, N]
    bias = torch.randn(72, device="cuda")
    n0 = K.launch_count()
    y = _unwrap(lt.Ops.scaled_matmul(lt.Tensor(a), lt.Tensor(b), 0.25, 0.5, bias=lt.Tensor(bias)))
    assert K.launch_count() > n0                                              # the native kernel ran
    ref = (a.double() @ b.double()) * 0.125 + bias.double()
    assert y.dtype == torch.float32 and float((y.double() - ref).norm() / ref.norm()) < 1e-5
