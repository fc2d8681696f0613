"""The allocation-free norm backward (`lt_norm_bwd_noalloc`) called through its exported C symbol.

Some callers of the library cannot ask for device memory while they run (they live inside another
framework's pool, or their memory budget is fixed at start-up).  For them the library offers one entry
point whose scratch lives in a fixed array inside the library image.  This test checks it against the
regular entry point, twice in a row so that stale scratch contents from the first call would show.
It is collected last on purpose: a run that stops at the first failure has then already run every
other test.
"""
import ctypes
from ctypes import c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu

_ARGS = [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
         c_int, c_int, c_void_p]


def _close(a, b, tol=1.5e-2):
    err = ((a.float() - b.float()).norm() / (b.float().norm() + 1e-6)).item()
    assert err < tol, err


@pytest.mark.parametrize("layer_norm", [False, True])
def test_noalloc_matches_regular_entry_point_twice(layer_norm):
    from litetorch_b200._native import cuda_lib
    from litetorch_b200.ops import kernels as K
    fn = cuda_lib().lt_norm_bwd_noalloc
    fn.argtypes = _ARGS
    fn.restype = c_int
    torch.manual_seed(0)
    stream = torch.cuda.current_stream().cuda_stream
    for call, (M, D) in enumerate([(777, 2048), (300, 1024)]):
        x = torch.randn(M, D, device="cuda").bfloat16()
        dy = torch.randn(M, D, device="cuda").bfloat16()
        dres = torch.randn(M, D, device="cuda").bfloat16()
        w = (1 + 0.1 * torch.randn(D, device="cuda")).bfloat16()
        b = (0.1 * torch.randn(D, device="cuda")).bfloat16() if layer_norm else None
        _, _, mean, rstd = K.norm_fwd(x, w, b, None, layer_norm=layer_norm)
        dx_ref, dw_ref, db_ref = K.norm_bwd(dy, x, w, mean, rstd, layer_norm=layer_norm, dres=dres)
        dx = torch.empty_like(x)
        dw = torch.empty(D, device="cuda", dtype=torch.bfloat16)
        db = torch.empty(D, device="cuda", dtype=torch.bfloat16) if layer_norm else None
        # fp32 reference of the same backward pass, by autograd on plain PyTorch
        xf = x.float().requires_grad_(True)
        wf = w.float().requires_grad_(True)
        bf = b.float().requires_grad_(True) if layer_norm else None
        if layer_norm:
            yf = torch.nn.functional.layer_norm(xf, (D,), wf, bf, 1e-5)
        else:
            yf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5) * wf
        yf.backward(dy.float())
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        free_before = torch.cuda.mem_get_info()[0]          # the driver's view: would also see a raw cudaMalloc
        rc = fn(1 if layer_norm else 0, dy.data_ptr(), x.data_ptr(), w.data_ptr(),
                mean.data_ptr() if mean is not None else None, rstd.data_ptr(), dres.data_ptr(), dx.data_ptr(),
                dw.data_ptr(), db.data_ptr() if db is not None else None, 0, 0, M, D, stream)
        assert rc == 0, rc
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        assert torch.cuda.mem_get_info()[0] == free_before
        _close(dx, xf.grad + dres.float())
        _close(dw, wf.grad)
        if layer_norm:
            _close(db, bf.grad)
        _close(dx, dx_ref)
        _close(dw, dw_ref)
        if layer_norm:
            _close(db, db_ref)
    K.check_status()


def test_noalloc_rejects_rows_beyond_the_maximum():
    from litetorch_b200._native import cuda_lib
    fn = cuda_lib().lt_norm_bwd_noalloc
    fn.argtypes = _ARGS
    fn.restype = c_int
    D = 8192
    x = torch.zeros(4, D, device="cuda", dtype=torch.bfloat16)
    w = torch.ones(D, device="cuda", dtype=torch.bfloat16)
    r = torch.ones(4, device="cuda")
    rc = fn(0, x.data_ptr(), x.data_ptr(), w.data_ptr(), None, r.data_ptr(), None, x.data_ptr(), w.data_ptr(), None, 0, 0,
            4, D, torch.cuda.current_stream().cuda_stream)
    assert rc == -100


def test_noalloc_rejects_missing_or_misaligned_pointers_without_launching():
    from litetorch_b200._native import cuda_lib
    from litetorch_b200.ops import kernels as K
    fn = cuda_lib().lt_norm_bwd_noalloc
    fn.argtypes = _ARGS
    fn.restype = c_int
    M, D = 16, 256
    x = torch.zeros(M + 1, D, device="cuda", dtype=torch.bfloat16)
    w = torch.ones(D, device="cuda", dtype=torch.bfloat16)
    r = torch.ones(M, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    # LayerNorm without its mean (and without db): an argument error, not a device fault
    assert fn(1, x.data_ptr(), x.data_ptr(), w.data_ptr(), None, r.data_ptr(), None, x.data_ptr(), w.data_ptr(), None, 0, 0, M, D, st) == -6
    # a required pointer missing
    assert fn(0, None, x.data_ptr(), w.data_ptr(), None, r.data_ptr(), None, x.data_ptr(), w.data_ptr(), None, 0, 0, M, D, st) == -6
    # a bf16 base that is not 16-byte aligned
    assert fn(0, x.data_ptr() + 2, x.data_ptr(), w.data_ptr(), None, r.data_ptr(), None, x.data_ptr(), w.data_ptr(), None, 0, 0, M, D, st) == -6
    torch.cuda.synchronize()
    K.check_status()
