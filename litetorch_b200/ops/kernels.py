"""ctypes front-end of the sm_100a kernels in liblt_cuda.so.

Every function takes torch CUDA tensors, launches on the current torch stream and returns torch
tensors.  No autograd here: `litetorch_b200.ops.functional` wraps these into autograd Functions and
`litetorch_b200.models` calls them directly from hand-written layer backward passes.
"""
from __future__ import annotations

import ctypes
from ctypes import c_void_p, c_int, c_longlong, c_float

import torch

from .._native import cuda_lib

_vp, _i, _ll, _f = c_void_p, c_int, c_longlong, c_float

_SIGS = {
    "lt_status_fetch": [],
    "lt_sm_count": [],
    "lt_set_wait_budget_cycles": [_ll, _ll],
    "lt_gemm_bf16": [_vp, _vp, _vp, _i, _i, _i, _ll, _ll, _ll, _i, _i, _i, _vp, _vp, _ll, _i, _i, _f, _i, _i, _vp],
    "lt_gemm_typed": [_i, _vp, _vp, _vp, _i, _i, _i, _ll, _ll, _ll, _i, _i, _i, _vp, _vp, _ll, _i, _i, _f, _vp],
    "lt_gemv_bf16": [_vp, _ll, _vp, _ll, _vp, _ll, _vp, _ll, _i, _i, _i, _vp],
    "lt_gemm_skinny_bf16": [_vp, _ll, _vp, _ll, _vp, _ll, _vp, _ll, _i, _i, _i, _vp],
    "lt_gemm_skinny_set_target": [_i, _i],
    "lt_gemm_e4m3": [_vp, _vp, _vp, _i, _i, _i, _ll, _ll, _ll, _i, _vp, _vp, _vp, _vp, _ll, _i, _f, _vp],
    "lt_quant_e4m3_rows": [_vp, _ll, _vp, _ll, _vp, _i, _i, _vp],
    "lt_quant_int8_tensor": [_vp, _i, _vp, _ll, _f, _vp],
    "lt_quant_int8_rows": [_vp, _i, _vp, _vp, _i, _i, _vp],
    "lt_gemm_set_tail_split": [_i],
    "lt_gemm_set_pair_mode": [_i],
    "lt_flash_bwd_set_trace": [_vp],
    "lt_flash_fwd_set_trace": [_vp],
    "lt_gemm_fp8_block": [_vp, _vp, _vp, _i, _i, _i, _ll, _ll, _ll, _vp, _vp, _i, _vp, _i, _vp],
    "lt_gemm_fp8_block_pair": [_vp, _vp, _vp, _i, _i, _i, _ll, _ll, _ll, _vp, _vp, _i, _vp, _vp],
    "lt_quant_fp8_1x128": [_vp, _ll, _vp, _ll, _vp, _i, _i, _vp],
    "lt_moe_router": [_vp, _i, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp],
    "lt_moe_router_bwd": [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp],
    "lt_dropout": [_vp, _vp, _ll, _i, _f, ctypes.c_ulonglong, ctypes.c_ulonglong, _vp],
    "lt_softmax_fwd": [_vp, _vp, _ll, _i, _i, _vp],
    "lt_softmax_bwd": [_vp, _vp, _vp, _ll, _i, _i, _vp],
    "lt_quant_fp8_128x128": [_vp, _ll, _vp, _ll, _vp, _i, _i, _vp],
    "lt_unscale_check": [_vp, _ll, _i, _f, _vp, _vp],
    "lt_reduce_parts": [],
    "lt_reduce_all": [_vp, _ll, _i, _i, _vp, _vp, _vp],
    "lt_strided_copy": [_vp, _vp, _i, _vp, _vp, _vp, _i, _vp],
    "lt_moe_expert_bwd": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _vp],
    "lt_norm_bwd_ctas": [_i],
    "lt_norm_fwd": [_i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _f, _vp],
    "lt_norm_bwd": [_i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp],
    "lt_rope": [_vp, _vp, _vp, _vp, _ll, _i, _i, _i, _ll, _i, _vp],
    "lt_swiglu_fwd": [_vp, _vp, _ll, _i, _vp],
    "lt_swiglu_bwd": [_vp, _vp, _vp, _ll, _i, _vp],
    "lt_gelu_fwd": [_vp, _vp, _ll, _vp],
    "lt_gelu_bwd": [_vp, _vp, _vp, _ll, _vp],
    "lt_axpby": [_vp, _vp, _vp, _f, _f, _ll, _vp],
    "lt_embedding_fwd": [_vp, _vp, _vp, _ll, _i, _i, _vp],
    "lt_embedding_bwd": [_vp, _vp, _vp, _ll, _i, _i, _vp],
    "lt_cast_f32_to_bf16": [_vp, _vp, _ll, _vp],
    "lt_cast_bf16_to_f32": [_vp, _vp, _ll, _vp],
    "lt_ce_stats": [_vp, _ll, _vp, _i, _i, _i, _vp, _vp],
    "lt_ce_finish": [_vp, _ll, _vp, _i, _i, _i, _vp, _vp, _f, _ll, _i, _vp],
    "lt_adam_flat": [_vp, _vp, _i, _vp, _vp, _vp, _ll, _f, _f, _f, _f, _f, _f, _f, _i, _vp, _vp],
    "lt_adam_table": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _f, _f, _f, _f, _f, _f, _f, _i, _vp, _vp],
    "lt_adam_chunk_elems": [],
    "lt_adam_q8": [_vp, _i, _vp, _i, _vp, _vp, _ll, _f, _f, _f, _f, _f, _f, _f, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp],
    "lt_sgd_flat": [_vp, _vp, _vp, _ll, _f, _f, _f, _vp],
    "lt_rmsprop_flat": [_vp, _vp, _vp, _ll, _f, _f, _f, _f, _vp],
    "lt_sumsq": [_vp, _i, _ll, _vp, _vp],
    "lt_clip_coef": [_vp, _vp, _f, _f, _vp],
    "lt_ag_gemm_bf16": [_vp, _vp, _vp, _i, _i, _i, _ll, _ll, _ll, _i, _i, _i, _vp, _vp, _ll, _i, _i, _f,
                        _i, _vp, _i, _i, _i, _vp, _vp, ctypes.c_uint, _i, _vp, _vp, ctypes.c_uint, _vp],
    "lt_rs_adamw": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _f, _f, _f, _f, _f, _f, _f, _vp, _vp, _i, ctypes.c_uint, _i, _i, _i, _vp],
    "lt_embedding_fwd_sharded": [_vp, _vp, _vp, _ll, _i, _i, _i, _i, _vp],
    "lt_signal_barrier": [_vp, _vp, _i, ctypes.c_uint, _i, _i, _vp],
    "lt_gather_shards": [_vp, _i, _vp, _vp, _i, _i, _vp],
    "lt_gemm_num_tiles": [_i, _i, _i],
    "lt_paged_decode": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _f, _i, _f, _f, _vp],
    "lt_kv_append": [_vp, _vp, _vp, _vp, _vp, _ll, _i, _i, _i, _i, _f, _f, _vp],
    "lt_gemm_rs_bf16": [_vp, _vp, _i, _i, _i, _ll, _ll, _i, _vp, _vp, ctypes.c_uint, _i, _i, _i, _vp, _ll, _vp, _vp, _ll, _vp],
    "lt_flash_fwd": [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _ll, _ll, _ll, _ll, _ll, _ll, _ll, _ll, _f, _i, _vp],
    "lt_moe_gather_gemm": [_vp, _i, _vp, _vp, _i, _vp, _i, _i, _i, _i, _vp, _vp, ctypes.c_uint, _vp, _vp, _i, _vp],
    "lt_moe_gemm_scatter": [_vp, _vp, _i, _vp, _i, _i, _i, _i, _vp, _vp, _vp, _i, _vp],
    "lt_flash_fwd_cp": [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _ll, _ll, _ll, _ll, _ll, _ll, _ll, _ll, _f, _i, _i, _i, _i, _vp],
    "lt_flash_bwd_cp": [_i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i,
                        _ll, _ll, _ll, _ll, _ll, _ll, _ll, _ll, _ll, _ll, _ll, _ll, _ll, _ll, _f, _i, _i, _i, _i, _vp],
    "lt_flash_bwd": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i,
                     _ll, _ll, _ll, _ll, _ll, _ll, _ll, _ll, _ll, _ll, _ll, _ll, _ll, _ll, _f, _i, _vp],
}

_bound = {}

# Kernels launched per native call; `launch_count()` is what bench.py reports as "gpu_launches".
_LAUNCHES_PER_CALL = {"lt_gemm_num_tiles": 0, "lt_gemm_skinny_set_target": 0, "lt_adam_q8": 3, "lt_set_wait_budget_cycles": 0, "lt_norm_bwd": 2, "lt_paged_decode": 2, "lt_flash_bwd": 3, "lt_status_fetch": 0, "lt_sm_count": 0, "lt_gemm_set_tail_split": 0, "lt_reduce_parts": 0, "lt_reduce_all": 2, "lt_gemm_set_pair_mode": 0, "lt_flash_bwd_set_trace": 0, "lt_flash_fwd_set_trace": 0, "lt_norm_bwd_ctas": 0,
                      "lt_adam_chunk_elems": 0}
_launches = [0]


def launch_count() -> int:
    return _launches[0]


def reset_launch_count():
    _launches[0] = 0


class KernelError(RuntimeError):
    pass


def _fn(name):
    f = _bound.get(name)
    if f is None:
        lib = cuda_lib()
        raw = getattr(lib, name)
        raw.argtypes = _SIGS[name]
        raw.restype = c_int
        n = _LAUNCHES_PER_CALL.get(name, 1)
        if n:
            def f(*a, _raw=raw, _n=n):
                _launches[0] += _n
                return _raw(*a)
        else:
            f = raw
        _bound[name] = f
    return f


def has_kernel(name: str) -> bool:
    try:
        return hasattr(cuda_lib(), name)
    except Exception:
        return False


def _check(rc, name):
    if rc != 0:
        raise KernelError("%s failed with code %d" % (name, rc))


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _p(t):
    return None if t is None else t.data_ptr()


def status_fetch() -> int:
    """Read-and-clear the device status word (synchronises). 0 = no bounded wait ran out."""
    return _fn("lt_status_fetch")()


def check_status():
    s = status_fetch()
    if s != 0:
        raise KernelError("device status word = %d (a bounded wait ran out or an argument was rejected)" % s)


def set_wait_budget(local_cycles: int = 0, peer_cycles: int = 0):
    """Clock budget (SM cycles) of the bounded waits inside the kernels on the current device: `local_cycles` for
    mbarriers and flags set on this GPU, `peer_cycles` for flags set by another GPU; 0 restores the defaults (about
    1.5 s / 10 s).  A wait that runs out records a code in the status word (`status_fetch`) and the kernel returns."""
    torch.cuda.synchronize()
    _check(_fn("lt_set_wait_budget_cycles")(int(local_cycles), int(peer_cycles)), "lt_set_wait_budget_cycles")


def sm_count() -> int:
    return _fn("lt_sm_count")()


# ------------------------------------------------------------------------------------------------ GEMM
def gemm(a: torch.Tensor, b: torch.Tensor, *, a_major: int = 0, b_major: int = 0, out: torch.Tensor | None = None,
         out_dtype=torch.bfloat16, bias=None, residual=None, act: int = 0, accumulate: bool = False,
         alpha: float = 1.0, block_n: int = 0, max_ctas: int = 0) -> torch.Tensor:
    """C = epilogue(alpha * op(A) @ op(B)).

    a_major=0: ``a`` is [M, K];  a_major=1: ``a`` is [K, M] (used transposed).
    b_major=0: ``b`` is [N, K];  b_major=1: ``b`` is [K, N].
    Rows may be strided (last dim contiguous).
    """
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and a.dim() == 2 and b.dim() == 2
    assert a.stride(1) == 1 and b.stride(1) == 1
    if (a_major == 0 and b_major == 0 and a.shape[0] <= 8 and out is None and out_dtype == torch.bfloat16 and bias is None and act == 0
            and alpha == 1.0 and a.shape[1] % 8 == 0 and a.stride(0) % 8 == 0 and b.stride(0) % 8 == 0 and a.shape[0] > 0
            and a.data_ptr() % 16 == 0 and b.data_ptr() % 16 == 0):
        # a handful of rows (decode): the weight-streaming kernel, one warp per output column
        M, Kd = a.shape
        N = b.shape[0]
        y = torch.empty((M, N), dtype=torch.bfloat16, device=a.device)
        rc = _fn("lt_gemv_bf16")(a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0), y.data_ptr(), y.stride(0), _p(residual),
                                 residual.stride(0) if residual is not None else 0, M, N, Kd, _stream())
        _check(rc, "lt_gemv_bf16")
        return y
    if (a_major == 0 and b_major == 0 and 8 < a.shape[0] <= 128 and out_dtype == torch.bfloat16 and bias is None and act == 0
            and alpha == 1.0 and not accumulate and a.shape[1] % 32 == 0 and b.shape[0] % 8 == 0 and a.stride(0) % 8 == 0
            and b.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0 and b.data_ptr() % 16 == 0 and a.shape[1] == b.shape[1]
            and (out is None or (out.dtype == torch.bfloat16 and out.shape == (a.shape[0], b.shape[0]) and out.stride(1) == 1
                                 and out.stride(0) % 2 == 0 and out.data_ptr() % 4 == 0))
            and (residual is None or (residual.dtype == torch.bfloat16 and residual.shape == (a.shape[0], b.shape[0])
                                      and residual.stride(1) == 1 and residual.stride(0) % 2 == 0 and residual.data_ptr() % 4 == 0))):
        # 9 to 128 rows (decode with a batch of sequences): the weight-streaming tensor-core kernel
        M, Kd = a.shape
        N = b.shape[0]
        y = out if out is not None else torch.empty((M, N), dtype=torch.bfloat16, device=a.device)
        rc = _fn("lt_gemm_skinny_bf16")(a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0), y.data_ptr(), y.stride(0), _p(residual),
                                        residual.stride(0) if residual is not None else 0, M, N, Kd, _stream())
        _check(rc, "lt_gemm_skinny_bf16")
        return y
    if a_major == 0:
        M, K = a.shape
    else:
        K, M = a.shape
    if b_major == 0:
        N, Kb = b.shape
    else:
        Kb, N = b.shape
    assert K == Kb, "inner dimensions differ: %d vs %d" % (K, Kb)
    if out is None:
        assert not accumulate
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    assert out.shape == (M, N) and out.stride(1) == 1 and out.dtype in (torch.bfloat16, torch.float32)
    if residual is not None:
        assert residual.dtype == torch.bfloat16 and residual.shape == (M, N) and residual.stride(1) == 1
    if bias is not None:
        assert bias.dtype == torch.bfloat16 and bias.numel() == N and bias.is_contiguous()
    rc = _fn("lt_gemm_bf16")(a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, a.stride(0), b.stride(0), out.stride(0),
                             a_major, b_major, 1 if out.dtype == torch.float32 else 0, _p(bias), _p(residual),
                             residual.stride(0) if residual is not None else 0, act, 1 if accumulate else 0,
                             float(alpha), block_n, max_ctas, _stream())
    _check(rc, "lt_gemm_bf16")
    return out


def gemm_any(a: torch.Tensor, b: torch.Tensor, *, a_major: int = 0, b_major: int = 0, out_dtype=None) -> torch.Tensor:
    """The tcgen05 GEMM for bf16, fp16 and fp32 operands (layouts as in `gemm`).  fp16 runs as kind::f16 with an fp32
    result that is rounded to fp16 afterwards; fp32 runs on the tensor cores as tf32 (both operands are brought to the
    K-major layout first) and returns fp32."""
    dt = a.dtype
    assert b.dtype == dt and a.dim() == 2 and b.dim() == 2
    if dt == torch.bfloat16:
        return gemm(a, b, a_major=a_major, b_major=b_major, out_dtype=out_dtype or torch.bfloat16)
    if dt == torch.float32:
        if a_major == 1:
            a, a_major = a.t().contiguous(), 0
        if b_major == 1:
            b, b_major = b.t().contiguous(), 0
        kind = 2
    elif dt == torch.float16:
        kind = 1
    else:
        raise TypeError("gemm_any: %s" % dt)
    a = a if a.stride(1) == 1 else a.contiguous()
    b = b if b.stride(1) == 1 else b.contiguous()
    M, Kd = a.shape if a_major == 0 else (a.shape[1], a.shape[0])
    N = b.shape[0] if b_major == 0 else b.shape[1]
    assert (b.shape[1] if b_major == 0 else b.shape[0]) == Kd, "inner dimensions differ"
    out = torch.empty((M, N), dtype=torch.float32, device=a.device)
    rc = _fn("lt_gemm_typed")(kind, a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, Kd, a.stride(0), b.stride(0), out.stride(0),
                              a_major, b_major, 1, None, None, 0, 0, 0, 1.0, _stream())
    _check(rc, "lt_gemm_typed")
    want = out_dtype or dt
    return out if want == torch.float32 else out.to(want)


def quant_int8_tensor(x: torch.Tensor, scale: float) -> torch.Tensor:
    """clamp(round(x / scale), -127, 127) as int8 (x fp32 or bf16, contiguous)."""
    x = x.contiguous()
    q = torch.empty(x.shape, dtype=torch.int8, device=x.device)
    _check(_fn("lt_quant_int8_tensor")(x.data_ptr(), _dt(x), q.data_ptr(), x.numel(), float(scale), _stream()), "lt_quant_int8_tensor")
    return q


def quant_int8_rows(x: torch.Tensor):
    """Per-row absmax int8 codes of a 2-D tensor: (q int8 [R, C], scale fp32 [R]) with x ~ q * scale[:, None]."""
    x = x.contiguous()
    R, C = x.shape
    q = torch.empty((R, C), dtype=torch.int8, device=x.device)
    sc = torch.empty(R, dtype=torch.float32, device=x.device)
    _check(_fn("lt_quant_int8_rows")(x.data_ptr(), _dt(x), q.data_ptr(), sc.data_ptr(), R, C, _stream()), "lt_quant_int8_rows")
    return q, sc


def gemm_i8(a: torch.Tensor, b: torch.Tensor, alpha: float = 1.0) -> torch.Tensor:
    """fp32 C[M, N] = alpha * (a[M, K] @ b[N, K]^T) for int8 operands with exact 32-bit integer accumulation on the
    tensor cores (tcgen05 kind::i8); K a multiple of 16."""
    assert a.dtype == torch.int8 and b.dtype == torch.int8 and a.dim() == 2 and b.dim() == 2 and a.shape[1] == b.shape[1]
    a, b = a.contiguous(), b.contiguous()
    M, Kd = a.shape
    N = b.shape[0]
    out = torch.empty((M, N), dtype=torch.float32, device=a.device)
    rc = _fn("lt_gemm_typed")(3, a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, Kd, a.stride(0), b.stride(0), out.stride(0),
                              0, 0, 1, None, None, 0, 0, 0, float(alpha), _stream())
    _check(rc, "lt_gemm_typed(int8)")
    return out


def gemm_set_tail_split(enable: bool):
    """Turn the K-split of the last, partly filled tile wave of `gemm` on (default) or off."""
    _fn("lt_gemm_set_tail_split")(1 if enable else 0)


def gemm_skinny_set_target(ctas_per_sm: int = 1, min_chunks_per_warp: int = 16):
    """Tuning of the 9-128-row weight-streaming GEMM on narrow outputs: CTAs per SM that its K split aims for and the
    fewest 32-element chunks of K a warp keeps (defaults 1 and 16: K is split from 8192 on)."""
    _fn("lt_gemm_skinny_set_target")(int(ctas_per_sm), int(min_chunks_per_warp))


def gemm_set_pair_mode(mode: int):
    """0: one CTA per tile only; 1 (default): CTA pairs (cta_group::2, 256 x 256 tiles) where the cost model
    prefers them; 2: CTA pairs for every shape."""
    _fn("lt_gemm_set_pair_mode")(int(mode))


def quant_e4m3_rows(x: torch.Tensor):
    """x [M, K] bf16 (K a multiple of 8, rows may be strided) -> (e4m3 codes [M, K], fp32 scales [M]): row r is divided by
    scale[r] = absmax(row r) / 448 before rounding, so x ~ codes * scale[:, None]."""
    M, Kd = x.shape
    assert x.dtype == torch.bfloat16 and x.stride(1) == 1 and Kd % 8 == 0
    q = torch.empty((M, Kd), dtype=torch.float8_e4m3fn, device=x.device)
    sc = torch.empty(M, dtype=torch.float32, device=x.device)
    rc = _fn("lt_quant_e4m3_rows")(x.data_ptr(), x.stride(0), q.data_ptr(), q.stride(0), sc.data_ptr(), M, Kd, _stream())
    _check(rc, "lt_quant_e4m3_rows")
    return q, sc


def gemm_e4m3(aq: torch.Tensor, a_scale, bq: torch.Tensor, b_scale, *, out=None, out_dtype=torch.bfloat16, bias=None, residual=None,
              act: int = 0, alpha: float = 1.0) -> torch.Tensor:
    """C[M, N] = epilogue((aq[M, K] @ bq[N, K]^T) * a_scale[:, None] * b_scale[None, :]) for e4m3 operands on tcgen05
    kind::f8f6f4 (CTA pairs, the whole K extent accumulated in tensor memory, scales applied once in the epilogue).
    a_scale [M] / b_scale [N] fp32 or None; K a multiple of 16."""
    assert aq.dtype == torch.float8_e4m3fn and bq.dtype == torch.float8_e4m3fn and aq.dim() == 2 and bq.dim() == 2
    assert aq.stride(1) == 1 and bq.stride(1) == 1 and aq.shape[1] == bq.shape[1]
    M, Kd = aq.shape
    N = bq.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=aq.device)
    assert out.shape == (M, N) and out.stride(1) == 1 and out.dtype in (torch.bfloat16, torch.float32)
    for sc, n in ((a_scale, M), (b_scale, N)):
        assert sc is None or (sc.dtype == torch.float32 and sc.numel() == n and sc.is_contiguous())
    if residual is not None:
        assert residual.dtype == torch.bfloat16 and residual.shape == (M, N) and residual.stride(1) == 1
    if bias is not None:
        assert bias.dtype == torch.bfloat16 and bias.numel() == N and bias.is_contiguous()
    rc = _fn("lt_gemm_e4m3")(aq.data_ptr(), bq.data_ptr(), out.data_ptr(), M, N, Kd, aq.stride(0), bq.stride(0), out.stride(0),
                             1 if out.dtype == torch.float32 else 0, _p(a_scale), _p(b_scale), _p(bias), _p(residual),
                             residual.stride(0) if residual is not None else 0, act, float(alpha), _stream())
    _check(rc, "lt_gemm_e4m3")
    return out


def quant_fp8_1x128(x):
    """x [M, K] bf16 (K a multiple of 128) -> (e4m3 codes [M, K], scales [K/128, M] fp32, K-block major)."""
    M, K = x.shape
    assert x.dtype == torch.bfloat16 and x.stride(1) == 1 and K % 128 == 0
    q = torch.empty(M, K, dtype=torch.float8_e4m3fn, device=x.device)
    st = torch.empty(K // 128, M, dtype=torch.float32, device=x.device)
    rc = _fn("lt_quant_fp8_1x128")(x.data_ptr(), x.stride(0), q.data_ptr(), q.stride(0), st.data_ptr(), M, K, _stream())
    _check(rc, "lt_quant_fp8_1x128")
    return q, st


def gemm_fp8_block(a8, a_scale_t, b8, b_scale, out=None, *, bias=None, out_dtype=torch.bfloat16, max_ctas=0, pairs=None):
    """out[M, N] = block-scaled a8[M, K] @ b8[N, K]^T.  a_scale_t: [K/128, M] fp32; b_scale: [ceil(N/128), K/128] fp32.
    pairs=True runs the CTA-pair variant (256 x 256 tiles on cta_group::2); measured slower than the one-CTA kernel
    (the promotion of 128 x 256 fp32 partials per K block out of tensor memory is the bound, not the operand traffic),
    so it is off unless asked for."""
    M, K = a8.shape
    N = b8.shape[0]
    assert a8.dtype == torch.float8_e4m3fn and b8.dtype == torch.float8_e4m3fn and b8.shape[1] == K
    assert a8.stride(1) == 1 and b8.stride(1) == 1 and K % 128 == 0
    assert a_scale_t.shape == (K // 128, M) and a_scale_t.is_contiguous() and a_scale_t.dtype == torch.float32
    assert b_scale.shape == ((N + 127) // 128, K // 128) and b_scale.is_contiguous() and b_scale.dtype == torch.float32
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype, device=a8.device)
    if pairs is None:
        pairs = False
    if pairs:
        rc = _fn("lt_gemm_fp8_block_pair")(a8.data_ptr(), b8.data_ptr(), out.data_ptr(), M, N, K, a8.stride(0), b8.stride(0),
                                           out.stride(0), a_scale_t.data_ptr(), b_scale.data_ptr(),
                                           1 if out.dtype == torch.float32 else 0, _p(bias), _stream())
        _check(rc, "lt_gemm_fp8_block_pair")
        return out
    rc = _fn("lt_gemm_fp8_block")(a8.data_ptr(), b8.data_ptr(), out.data_ptr(), M, N, K, a8.stride(0), b8.stride(0),
                                  out.stride(0), a_scale_t.data_ptr(), b_scale.data_ptr(),
                                  1 if out.dtype == torch.float32 else 0, _p(bias), max_ctas, _stream())
    _check(rc, "lt_gemm_fp8_block")
    return out


# ------------------------------------------------------------------------------------------------ norms
def norm_fwd(x, weight, bias=None, residual=None, *, layer_norm=False, eps=1e-5, want_sum=True, out=None):
    """Returns (y, sum_or_None, mean_or_None, rstd).  x, residual: [M, D] bf16.  `out`: optional contiguous [M, D]
    buffer for y (e.g. the symmetric-memory slot a tensor-parallel gather reads from)."""
    M, D = x.shape
    y = torch.empty_like(x) if out is None else out
    assert y.shape == x.shape and y.is_contiguous() and y.dtype == x.dtype
    s = torch.empty_like(x) if (residual is not None and want_sum) else None
    mean = torch.empty(M, dtype=torch.float32, device=x.device) if layer_norm else None
    rstd = torch.empty(M, dtype=torch.float32, device=x.device)
    rc = _fn("lt_norm_fwd")(1 if layer_norm else 0, x.data_ptr(), _p(residual), weight.data_ptr(), _p(bias), y.data_ptr(),
                            _p(s), _p(mean), rstd.data_ptr(), M, D, float(eps), _stream())
    _check(rc, "lt_norm_fwd")
    return y, s, mean, rstd


def norm_bwd(dy, x, weight, mean, rstd, *, layer_norm=False, dres=None, dw=None, db=None, accumulate=False, out=None):
    """Returns (dx, dw, db).  `x` is the tensor that was normalised (the residual sum when one was fused).
    `out`: optional contiguous [M, D] buffer for dx."""
    M, D = x.shape
    dx = torch.empty_like(x) if out is None else out
    assert dx.shape == x.shape and dx.is_contiguous() and dx.dtype == x.dtype
    ctas = _fn("lt_norm_bwd_ctas")(M)
    part = torch.empty((2 if layer_norm else 1, ctas, D), dtype=torch.float32, device=x.device)
    if dw is None:
        dw = torch.empty(D, dtype=weight.dtype, device=x.device)
        accumulate = False
    if layer_norm and db is None:
        db = torch.empty(D, dtype=weight.dtype, device=x.device)
    rc = _fn("lt_norm_bwd")(1 if layer_norm else 0, dy.data_ptr(), x.data_ptr(), weight.data_ptr(), _p(mean), rstd.data_ptr(),
                            _p(dres), dx.data_ptr(), part[0].data_ptr(), part[1].data_ptr() if layer_norm else None,
                            dw.data_ptr(), _p(db) if layer_norm else None, 1 if dw.dtype == torch.float32 else 0,
                            1 if accumulate else 0, M, D, _stream())
    _check(rc, "lt_norm_bwd")
    return dx, dw, db


# ------------------------------------------------------------------------------------------------ pointwise
def rope_(x2d: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, T: int, heads: int, head_dim: int, *,
          col_offset: int = 0, positions: torch.Tensor | None = None, backward: bool = False):
    """In-place interleaved-pair rotation of `heads` heads starting at column `col_offset` of a [rows, pitch] buffer."""
    rows = x2d.shape[0]
    base = x2d.data_ptr() + col_offset * x2d.element_size()
    rc = _fn("lt_rope")(base, cos.data_ptr(), sin.data_ptr(), _p(positions), rows, T, heads, head_dim, x2d.stride(0),
                        1 if backward else 0, _stream())
    _check(rc, "lt_rope")
    return x2d


def swiglu_fwd(gu: torch.Tensor) -> torch.Tensor:
    M, F2 = gu.shape
    h = torch.empty((M, F2 // 2), dtype=gu.dtype, device=gu.device)
    _check(_fn("lt_swiglu_fwd")(gu.data_ptr(), h.data_ptr(), M, F2 // 2, _stream()), "lt_swiglu_fwd")
    return h


def swiglu_bwd(gu: torch.Tensor, dh: torch.Tensor, inplace: bool = True) -> torch.Tensor:
    M, F2 = gu.shape
    dgu = gu if inplace else torch.empty_like(gu)
    _check(_fn("lt_swiglu_bwd")(gu.data_ptr(), dh.data_ptr(), dgu.data_ptr(), M, F2 // 2, _stream()), "lt_swiglu_bwd")
    return dgu


def gelu_fwd(x):
    y = torch.empty_like(x)
    _check(_fn("lt_gelu_fwd")(x.data_ptr(), y.data_ptr(), x.numel(), _stream()), "lt_gelu_fwd")
    return y


def gelu_bwd(x, dy):
    dx = torch.empty_like(x)
    _check(_fn("lt_gelu_bwd")(x.data_ptr(), dy.data_ptr(), dx.data_ptr(), x.numel(), _stream()), "lt_gelu_bwd")
    return dx


def axpby(a, b=None, alpha=1.0, beta=1.0, out=None):
    out = torch.empty_like(a) if out is None else out
    _check(_fn("lt_axpby")(a.data_ptr(), _p(b), out.data_ptr(), float(alpha), float(beta), a.numel(), _stream()), "lt_axpby")
    return out


def embedding_fwd(idx: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    idx = idx.reshape(-1).to(torch.int64)
    V, D = table.shape
    out = torch.empty((idx.numel(), D), dtype=table.dtype, device=table.device)
    _check(_fn("lt_embedding_fwd")(idx.data_ptr(), table.data_ptr(), out.data_ptr(), idx.numel(), D, V, _stream()), "lt_embedding_fwd")
    return out


def embedding_bwd(idx: torch.Tensor, dout: torch.Tensor, dtable: torch.Tensor):
    idx = idx.reshape(-1).to(torch.int64)
    V, D = dtable.shape
    _check(_fn("lt_embedding_bwd")(idx.data_ptr(), dout.data_ptr(), dtable.data_ptr(), idx.numel(), D, V, _stream()), "lt_embedding_bwd")
    return dtable


def cast_to_bf16(x: torch.Tensor, out=None):
    out = torch.empty(x.shape, dtype=torch.bfloat16, device=x.device) if out is None else out
    _check(_fn("lt_cast_f32_to_bf16")(x.data_ptr(), out.data_ptr(), x.numel(), _stream()), "lt_cast_f32_to_bf16")
    return out


def cast_to_f32(x: torch.Tensor, out=None):
    out = torch.empty(x.shape, dtype=torch.float32, device=x.device) if out is None else out
    _check(_fn("lt_cast_bf16_to_f32")(x.data_ptr(), out.data_ptr(), x.numel(), _stream()), "lt_cast_bf16_to_f32")
    return out


# ------------------------------------------------------------------------------------------------ loss
def ce_stats(logits: torch.Tensor, targets: torch.Tensor, vocab_start: int = 0) -> torch.Tensor:
    N, V = logits.shape
    stats = torch.empty((N, 3), dtype=torch.float32, device=logits.device)
    _check(_fn("lt_ce_stats")(logits.data_ptr(), logits.stride(0), targets.data_ptr(), vocab_start, N, V, stats.data_ptr(), _stream()), "lt_ce_stats")
    return stats


def ce_finish(logits, targets, gstats, *, vocab_start=0, grad_scale=1.0, ignore_index=-100, write_grad=True):
    """Per-row losses; overwrites `logits` with d(loss)/d(logits) * grad_scale when write_grad."""
    N, V = logits.shape
    loss = torch.empty(N, dtype=torch.float32, device=logits.device)
    _check(_fn("lt_ce_finish")(logits.data_ptr(), logits.stride(0), targets.data_ptr(), vocab_start, N, V, gstats.data_ptr(),
                               loss.data_ptr(), float(grad_scale), ignore_index, 1 if write_grad else 0, _stream()), "lt_ce_finish")
    return loss


# ------------------------------------------------------------------------------------------------ optimizers
def adam_flat(master, grad, m, v, param_bf16, *, lr, beta1, beta2, eps, wd, step, adamw=True, dyn=None):
    bc1 = 1.0 - beta1 ** step
    bc2 = 1.0 - beta2 ** step
    _check(_fn("lt_adam_flat")(master.data_ptr(), grad.data_ptr(), 1 if grad.dtype == torch.bfloat16 else 0, m.data_ptr(),
                               v.data_ptr(), _p(param_bf16), master.numel(), lr, beta1, beta2, eps, wd, bc1, bc2,
                               1 if adamw else 0, _p(dyn), _stream()), "lt_adam_flat")


def sgd_flat(p, g, vel, *, lr, momentum, wd):
    """p -= lr * (momentum * vel + g + wd * p) on contiguous fp32 tensors (vel None: no momentum)."""
    _check(_fn("lt_sgd_flat")(p.data_ptr(), g.data_ptr(), _p(vel), p.numel(), lr, momentum, wd, _stream()), "lt_sgd_flat")


def rmsprop_flat(p, g, sq, *, lr, alpha, eps, wd):
    _check(_fn("lt_rmsprop_flat")(p.data_ptr(), g.data_ptr(), sq.data_ptr(), p.numel(), lr, alpha, eps, wd, _stream()), "lt_rmsprop_flat")


def adam_q8(p, g, mq, vq, *, lr, beta1, beta2, eps, wd, step, fp8, first, scale_old, scale_new, amax, hist, hist_n):
    """AdamW step with int8 / e4m3 moment codes; scales, absmax and history stay on the device (no host sync)."""
    _check(_fn("lt_adam_q8")(p.data_ptr(), 1 if p.dtype == torch.bfloat16 else 0, g.data_ptr(), 1 if g.dtype == torch.bfloat16 else 0,
                             mq.data_ptr(), vq.data_ptr(), p.numel(), lr, beta1, beta2, eps, wd, 1.0 - beta1 ** step,
                             1.0 - beta2 ** step, 1 if fp8 else 0, 1 if first else 0, scale_old.data_ptr(), scale_new.data_ptr(),
                             amax.data_ptr(), hist.data_ptr(), hist_n.data_ptr(), _stream()), "lt_adam_q8")


def sumsq(x: torch.Tensor, out: torch.Tensor):
    _check(_fn("lt_sumsq")(x.data_ptr(), 1 if x.dtype == torch.bfloat16 else 0, x.numel(), out.data_ptr(), _stream()), "lt_sumsq")
    return out


def clip_coef(stats: torch.Tensor, dyn: torch.Tensor, max_norm: float, inv_scale: float = 1.0):
    _check(_fn("lt_clip_coef")(stats.data_ptr(), dyn.data_ptr(), float(max_norm), float(inv_scale), _stream()), "lt_clip_coef")
    return dyn


# ------------------------------------------------------------------------------------------------ attention
def flash_fwd(q, k, v, *, causal=True, scale=None):
    """q: [B, Tq, Hq, D], k/v: [B, Tk, Hkv, D] (last dim contiguous, arbitrary other strides).  Returns (o, lse)."""
    B, Tq, Hq, D = q.shape
    _, Tk, Hkv, _ = k.shape
    scale = (D ** -0.5) if scale is None else scale
    o = torch.empty((B, Tq, Hq, D), dtype=q.dtype, device=q.device)
    lse = torch.empty((B, Hq, Tq), dtype=torch.float32, device=q.device)
    rc = _fn("lt_flash_fwd")(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(), B, Tq, Tk, Hq, Hkv, D,
                             q.stride(0), q.stride(1), k.stride(0), k.stride(1), v.stride(0), v.stride(1),
                             o.stride(0), o.stride(1), float(scale), 1 if causal else 0, _stream())
    _check(rc, "lt_flash_fwd")
    return o, lse


def flash_bwd(q, k, v, o, lse, do, *, causal=True, scale=None, dq=None, dk=None, dv=None):
    """Returns (dq, dk, dv) with the shapes/strides of the given outputs (allocated contiguous when None)."""
    B, Tq, Hq, D = q.shape
    _, Tk, Hkv, _ = k.shape
    scale = (D ** -0.5) if scale is None else scale
    dq = torch.empty((B, Tq, Hq, D), dtype=q.dtype, device=q.device) if dq is None else dq
    dk = torch.empty((B, Tk, Hkv, D), dtype=q.dtype, device=q.device) if dk is None else dk
    dv = torch.empty((B, Tk, Hkv, D), dtype=q.dtype, device=q.device) if dv is None else dv
    delta = torch.empty((B, Hq, Tq), dtype=torch.float32, device=q.device)
    dq_acc = torch.zeros((B, Tq, Hq, D), dtype=torch.float32, device=q.device)
    rc = _fn("lt_flash_bwd")(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(), do.data_ptr(),
                             dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), delta.data_ptr(), dq_acc.data_ptr(),
                             B, Tq, Tk, Hq, Hkv, D,
                             q.stride(0), q.stride(1), k.stride(0), k.stride(1), v.stride(0), v.stride(1),
                             o.stride(0), o.stride(1), do.stride(0), do.stride(1),
                             dq.stride(0), dq.stride(1), dk.stride(0), dk.stride(1),
                             float(scale), 1 if causal else 0, _stream())
    _check(rc, "lt_flash_bwd")
    return dq, dk, dv


# ------------------------------------------------------------------------------------------------ fused communication
def _ptr_array(ptrs):
    arr = (c_void_p * len(ptrs))(*[int(p) for p in ptrs])
    return arr


class NextGather(ctypes.Structure):
    """The next gather-GEMM of the layer sequence, prefetched by the gather CTAs of the current one."""
    _fields_ = [("gather_operand", c_int), ("M", c_int), ("N", c_int), ("K", c_int), ("rows_per_rank", c_int), ("pad", c_int),
                ("shard_ptrs", c_void_p * 8), ("full", c_void_p), ("flags", c_void_p), ("epoch", ctypes.c_uint), ("pad2", ctypes.c_uint)]


def make_next_gather(gather_operand, M, N, Kd, rows_per_rank, shard_ptrs, full, flags, epoch) -> NextGather:
    ng = NextGather()
    ng.gather_operand, ng.M, ng.N, ng.K, ng.rows_per_rank = gather_operand, M, N, Kd, rows_per_rank
    for i, p in enumerate(shard_ptrs):
        ng.shard_ptrs[i] = int(p)
    ng.full, ng.flags, ng.epoch = full.data_ptr(), flags.data_ptr(), epoch
    return ng


def ag_gemm(a, b_full_or_a_full, *, gather_operand: int, shard_ptrs, world: int, rank: int, rows_per_rank: int,
            flags: torch.Tensor, epoch: int, other: torch.Tensor, out=None, out_dtype=torch.bfloat16, bias=None,
            residual=None, act: int = 0, accumulate: bool = False, alpha: float = 1.0, n_comm: int = 0,
            next_gather: "NextGather | None" = None, progress: "torch.Tensor | None" = None, progress_base: int = 0):
    """GEMM whose gathered operand is pulled from the ranks' shards by gather CTAs of the same kernel.

    gather_operand 1: C = other[M,K] @ full[N,K]^T      (full = weight gathered by rows, tiles gated by N block)
    gather_operand 2: C = other[M,K] @ full[K,N]        (full = weight [K rows, N], gated by K block)
    gather_operand 0: C = full[M,K] @ other[N,K]^T      (full = activation gathered by rows, gated by M block)
    `b_full_or_a_full` is the local staging buffer the shards are assembled in.
    """
    full = b_full_or_a_full
    if gather_operand == 0:
        A, B, a_major, b_major = full, other, 0, 0
        M, Kd = full.shape
        N = other.shape[0]
    elif gather_operand == 1:
        A, B, a_major, b_major = other, full, 0, 0
        M, Kd = other.shape
        N = full.shape[0]
    else:
        A, B, a_major, b_major = other, full, 0, 1
        M, Kd = other.shape
        N = full.shape[1]
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=other.device)
    arr = _ptr_array(shard_ptrs)
    rc = _fn("lt_ag_gemm_bf16")(A.data_ptr(), B.data_ptr(), out.data_ptr(), M, N, Kd, A.stride(0), B.stride(0), out.stride(0),
                                a_major, b_major, 1 if out.dtype == torch.float32 else 0, _p(bias), _p(residual),
                                residual.stride(0) if residual is not None else 0, act, 1 if accumulate else 0, float(alpha),
                                gather_operand, ctypes.cast(arr, c_void_p), world, rank, rows_per_rank, full.data_ptr(),
                                flags.data_ptr(), epoch, n_comm,
                                ctypes.cast(ctypes.pointer(next_gather), c_void_p) if next_gather is not None else None,
                                _p(progress), progress_base, _stream())
    _check(rc, "lt_ag_gemm_bf16")
    return out


def rs_adamw(grad_ptrs, mc_grads, master, m, v, param_shard, segs, *, lr, beta1, beta2, eps, wd, step, my_flags, peer_flag_ptrs,
             slot: int, epoch: int, world: int, rank: int, max_ctas: int = 0):
    seg_arr = (c_longlong * (3 * len(segs)))(*[int(x) for s in segs for x in s])
    rc = _fn("lt_rs_adamw")(ctypes.cast(_ptr_array(grad_ptrs), c_void_p), mc_grads, master.data_ptr(), m.data_ptr(), v.data_ptr(),
                            param_shard.data_ptr(), ctypes.cast(seg_arr, c_void_p), len(segs), lr, beta1, beta2, eps, wd,
                            1.0 - beta1 ** step, 1.0 - beta2 ** step, my_flags.data_ptr(),
                            ctypes.cast(_ptr_array(peer_flag_ptrs), c_void_p), slot, epoch, world, rank, max_ctas, _stream())
    _check(rc, "lt_rs_adamw")


def embedding_fwd_sharded(idx, table_ptrs, V, D, rows_per_rank, world, dtype=torch.bfloat16):
    idx = idx.reshape(-1).to(torch.int64)
    out = torch.empty((idx.numel(), D), dtype=dtype, device=idx.device)
    rc = _fn("lt_embedding_fwd_sharded")(idx.data_ptr(), ctypes.cast(_ptr_array(table_ptrs), c_void_p), out.data_ptr(),
                                         idx.numel(), D, V, rows_per_rank, world, _stream())
    _check(rc, "lt_embedding_fwd_sharded")
    return out


def gather_shards(shard_ptrs, segs, dsts, max_ctas: int = 0):
    """All-gather of row shards by peer loads.  segs: (shard_off, n) element pairs; dsts: one local tensor per segment
    that receives every rank's `n` elements in rank order (world * n elements)."""
    world = len(shard_ptrs)
    seg_arr = (c_longlong * (3 * len(segs)))(*[int(x) for s in segs for x in (s[0], s[1], 0)])
    rc = _fn("lt_gather_shards")(ctypes.cast(_ptr_array(shard_ptrs), c_void_p), world, ctypes.cast(seg_arr, c_void_p),
                                 ctypes.cast(_ptr_array([d.data_ptr() for d in dsts]), c_void_p), len(segs), max_ctas, _stream())
    _check(rc, "lt_gather_shards")


def signal_barrier(my_flags, peer_flag_ptrs, slot: int, epoch: int, world: int, rank: int):
    rc = _fn("lt_signal_barrier")(my_flags.data_ptr(), ctypes.cast(_ptr_array(peer_flag_ptrs), c_void_p), slot, epoch, world,
                                  rank, _stream())
    _check(rc, "lt_signal_barrier")


# ------------------------------------------------------------------------------------------------ serving
def paged_decode(q, k_cache, v_cache, block_tables, context_lens, block_size: int, splits: int, scale: float,
                 k_scale: float = 1.0, v_scale: float = 1.0):
    S, H, D = q.shape
    Hkv = k_cache.shape[1]
    part = torch.empty((S, H, splits, D + 2), dtype=torch.float32, device=q.device)
    o = torch.empty_like(q)
    rc = _fn("lt_paged_decode")(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), block_tables.data_ptr(),
                                context_lens.data_ptr(), part.data_ptr(), o.data_ptr(), S, H, Hkv, D, block_size,
                                block_tables.shape[1], k_cache.shape[0] if k_cache.is_contiguous() and v_cache.is_contiguous() else 0, splits,
                                float(scale), 1 if k_cache.dtype == torch.float8_e4m3fn else 0,
                                float(k_scale), float(v_scale), _stream())
    _check(rc, "lt_paged_decode")
    return o


def kv_append(k_new, v_new, k_cache, v_cache, slots, block_size: int, fp8: bool, k_scale: float = 1.0, v_scale: float = 1.0):
    N, Hkv, D = k_new.shape
    rc = _fn("lt_kv_append")(k_new.data_ptr(), v_new.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), slots.data_ptr(), N, Hkv, D,
                             block_size, 1 if fp8 else 0, float(k_scale), float(v_scale), _stream())
    _check(rc, "lt_kv_append")


def gemm_rs(a, b, *, b_major: int, stage_ptrs, counter_ptrs, epoch: int, world: int, rank: int, out=None, bias=None, residual=None):
    """out[M/world, N] = reduce-scatter over ranks of (a[M, K_local] @ op(b)), fused into the GEMM epilogue.
    b_major 0: b is [N, K_local]; 1: b is [K_local, N]."""
    M, Kd = a.shape
    N = b.shape[0] if b_major == 0 else b.shape[1]
    rpr = M // world
    if out is None:
        out = torch.empty((rpr, N), dtype=torch.bfloat16, device=a.device)
    rc = _fn("lt_gemm_rs_bf16")(a.data_ptr(), b.data_ptr(), M, N, Kd, a.stride(0), b.stride(0), b_major,
                                ctypes.cast(_ptr_array(stage_ptrs), c_void_p), ctypes.cast(_ptr_array(counter_ptrs), c_void_p),
                                epoch, world, rank, rpr, out.data_ptr(), out.stride(0), _p(bias), _p(residual),
                                residual.stride(0) if residual is not None else 0, _stream())
    _check(rc, "lt_gemm_rs_bf16")
    return out


def gemm_num_tiles(M: int, N: int, n_comm: int = 0) -> int:
    """Output tiles the GEMM launcher will use for an M x N result when `n_comm` SMs are set aside."""
    return _fn("lt_gemm_num_tiles")(M, N, n_comm)


# ------------------------------------------------------------------------------------------------ context-parallel attention
def flash_fwd_cp(q, k_ptrs, v_ptrs, k_like, *, causal, scale, cp_world, cp_rank, zigzag):
    """q: local queries [B, Tq, Hq, D]; k_ptrs / v_ptrs: every rank's KV shard (device pointers, layout of `k_like`)."""
    B, Tq, Hq, D = q.shape
    _, Tk, Hkv, _ = k_like.shape
    o = torch.empty((B, Tq, Hq, D), dtype=q.dtype, device=q.device)
    lse = torch.empty((B, Hq, Tq), dtype=torch.float32, device=q.device)
    rc = _fn("lt_flash_fwd_cp")(q.data_ptr(), ctypes.cast(_ptr_array(k_ptrs), c_void_p), ctypes.cast(_ptr_array(v_ptrs), c_void_p),
                                o.data_ptr(), lse.data_ptr(), B, Tq, Tk, Hq, Hkv, D, q.stride(0), q.stride(1), k_like.stride(0),
                                k_like.stride(1), k_like.stride(0), k_like.stride(1), o.stride(0), o.stride(1), float(scale),
                                1 if causal else 0, cp_world, cp_rank, 1 if zigzag else 0, _stream())
    _check(rc, "lt_flash_fwd_cp")
    return o, lse


def flash_bwd_cp(phase, *, q_ptrs, k, v, o, do_ptrs, lse_ptrs, delta_ptrs, dq_acc_ptrs, dq, dk, dv, q_like, causal, scale,
                 cp_world, cp_rank, zigzag):
    B, Tq, Hq, D = q_like.shape
    _, Tk, Hkv, _ = k.shape
    rc = _fn("lt_flash_bwd_cp")(phase, ctypes.cast(_ptr_array(q_ptrs), c_void_p), k.data_ptr(), v.data_ptr(), _p(o),
                                ctypes.cast(_ptr_array(do_ptrs), c_void_p), ctypes.cast(_ptr_array(lse_ptrs), c_void_p),
                                ctypes.cast(_ptr_array(delta_ptrs), c_void_p), ctypes.cast(_ptr_array(dq_acc_ptrs), c_void_p),
                                _p(dq), _p(dk), _p(dv), B, Tq, Tk, Hq, Hkv, D, q_like.stride(0), q_like.stride(1), k.stride(0),
                                k.stride(1), v.stride(0), v.stride(1), q_like.stride(0), q_like.stride(1), q_like.stride(0),
                                q_like.stride(1), q_like.stride(0), q_like.stride(1), k.stride(0), k.stride(1), float(scale),
                                1 if causal else 0, cp_world, cp_rank, 1 if zigzag else 0, _stream())
    _check(rc, "lt_flash_bwd_cp")


# ------------------------------------------------------------------------------------------------ mixture of experts
def moe_gather_gemm(src_ptrs, world, slot_src, group_of_mblk, weights, *, b_major, slot_buf, flags, epoch, row_scale=None,
                    n_comm=0):
    """out[slots, N] = rows fetched from the ranks' token buffers by `slot_src` @ op(weights[expert of the slot block])."""
    slots = slot_src.shape[0]
    E = weights.shape[0]
    N, Kd = (weights.shape[1], weights.shape[2]) if b_major == 0 else (weights.shape[2], weights.shape[1])
    out = torch.empty((slots, N), dtype=torch.bfloat16, device=weights.device)
    rc = _fn("lt_moe_gather_gemm")(ctypes.cast(_ptr_array(src_ptrs), c_void_p), world, slot_src.data_ptr(), group_of_mblk.data_ptr(),
                                   slots, weights.data_ptr(), E, N, Kd, b_major, slot_buf.data_ptr(), flags.data_ptr(), epoch,
                                   out.data_ptr(), _p(row_scale), n_comm, _stream())
    _check(rc, "lt_moe_gather_gemm")
    return out


def moe_gemm_scatter(a, group_of_mblk, weights, *, b_major, slot_dst, row_weight, acc_ptrs, world):
    """acc[dst rank][dst row] += row_weight * (a[slot] @ op(weights[expert])) with red.add into the owners' accumulators."""
    slots, Kd = a.shape
    E = weights.shape[0]
    N = weights.shape[1] if b_major == 0 else weights.shape[2]
    rc = _fn("lt_moe_gemm_scatter")(a.data_ptr(), group_of_mblk.data_ptr(), slots, weights.data_ptr(), E, N, Kd, b_major,
                                    slot_dst.data_ptr(), _p(row_weight), ctypes.cast(_ptr_array(acc_ptrs), c_void_p), world, _stream())
    _check(rc, "lt_moe_gemm_scatter")


# ------------------------------------------------------------------------------------------------ router, dropout, softmax ...
def _dt(t):
    if t.dtype == torch.float32:
        return 0
    if t.dtype == torch.bfloat16:
        return 1
    raise TypeError("expected float32 or bfloat16, got %s" % t.dtype)


def moe_router(logits, top_k: int, *, renorm: bool = True, counts=None, mass=None):
    """logits [N, E] (fp32 / bf16) -> (probs [N, E] fp32, topk_w [N, k] fp32, topk_idx [N, k] int32).
    counts [E] int32 and mass [E] fp32 are accumulated into when given (load-balancing statistics)."""
    N, E = logits.shape
    logits = logits.contiguous()
    probs = torch.empty(N, E, dtype=torch.float32, device=logits.device)
    tw = torch.empty(N, top_k, dtype=torch.float32, device=logits.device)
    ti = torch.empty(N, top_k, dtype=torch.int32, device=logits.device)
    rc = _fn("lt_moe_router")(logits.data_ptr(), _dt(logits), probs.data_ptr(), tw.data_ptr(), ti.data_ptr(), _p(counts),
                              _p(mass), N, E, top_k, 1 if renorm else 0, _stream())
    _check(rc, "lt_moe_router")
    return probs, tw, ti


def moe_router_bwd(probs, topk_idx, topk_w, d_topk_w, d_probs=None, *, renorm: bool = True):
    """Gradient of the router logits [N, E] fp32 from d(topk_w) and, optionally, a dense d(probs)."""
    N, E = probs.shape
    k = topk_idx.shape[1]
    dl = torch.empty(N, E, dtype=torch.float32, device=probs.device)
    d_topk_w = d_topk_w.contiguous().float()
    if d_probs is not None:
        d_probs = d_probs.contiguous().float()
    rc = _fn("lt_moe_router_bwd")(probs.data_ptr(), topk_idx.data_ptr(), topk_w.data_ptr(), d_topk_w.data_ptr(), _p(d_probs),
                                  dl.data_ptr(), N, E, k, 1 if renorm else 0, _stream())
    _check(rc, "lt_moe_router_bwd")
    return dl


def dropout(x, p: float, seed: int, offset: int = 0, out=None):
    """y = x * keep / (1 - p) with a Philox mask that depends only on (seed, offset, element index); the same call on
    the upstream gradient is the backward pass."""
    x = x.contiguous()
    y = torch.empty_like(x) if out is None else out
    rc = _fn("lt_dropout")(x.data_ptr(), y.data_ptr(), x.numel(), _dt(x), float(p), int(seed) & (2 ** 64 - 1),
                           int(offset) & (2 ** 64 - 1), _stream())
    _check(rc, "lt_dropout")
    return y


def softmax_fwd(x):
    """Softmax over the last dimension of a contiguous fp32 / bf16 tensor."""
    x = x.contiguous()
    y = torch.empty_like(x)
    D = x.shape[-1]
    rc = _fn("lt_softmax_fwd")(x.data_ptr(), y.data_ptr(), x.numel() // D, D, _dt(x), _stream())
    _check(rc, "lt_softmax_fwd")
    return y


def softmax_bwd(y, dy):
    y, dy = y.contiguous(), dy.contiguous()
    dx = torch.empty_like(y)
    D = y.shape[-1]
    rc = _fn("lt_softmax_bwd")(y.data_ptr(), dy.data_ptr(), dx.data_ptr(), y.numel() // D, D, _dt(y), _stream())
    _check(rc, "lt_softmax_bwd")
    return dx


def quant_fp8_128x128(w):
    """w [N, K] bf16 (K a multiple of 128) -> (e4m3 codes [N, K], scales [ceil(N/128), K/128] fp32)."""
    N, K = w.shape
    assert w.dtype == torch.bfloat16 and w.stride(1) == 1 and K % 128 == 0
    q = torch.empty(N, K, dtype=torch.float8_e4m3fn, device=w.device)
    sc = torch.empty((N + 127) // 128, K // 128, dtype=torch.float32, device=w.device)
    rc = _fn("lt_quant_fp8_128x128")(w.data_ptr(), w.stride(0), q.data_ptr(), q.stride(0), sc.data_ptr(), N, K, _stream())
    _check(rc, "lt_quant_fp8_128x128")
    return q, sc


def unscale_check_(g, inv_scale: float, found_inf):
    """g *= inv_scale in place; found_inf (int32 device scalar) is set to 1 if g held an inf or a nan."""
    assert g.is_contiguous() and found_inf.dtype == torch.int32
    rc = _fn("lt_unscale_check")(g.data_ptr(), g.numel(), _dt(g), float(inv_scale), found_inf.data_ptr(), _stream())
    _check(rc, "lt_unscale_check")
    return g


_reduce_scratch = {}


def reduce_all(x, mode: str = "sum"):
    """Sum or maximum of every element of a contiguous fp32 / bf16 tensor -> fp32 tensor of shape [1]."""
    x = x.contiguous()
    key = x.device
    part = _reduce_scratch.get(key)
    if part is None:
        part = torch.empty(_fn("lt_reduce_parts")(), dtype=torch.float32, device=x.device)
        _reduce_scratch[key] = part
    out = torch.empty(1, dtype=torch.float32, device=x.device)
    rc = _fn("lt_reduce_all")(x.data_ptr(), x.numel(), _dt(x), 1 if mode == "max" else 0, part.data_ptr(), out.data_ptr(),
                              _stream())
    _check(rc, "lt_reduce_all")
    return out


def strided_copy(src, dst):
    """dst[...] = src[...] for two views of the same shape (<= 8 dimensions, same element size): the gather behind
    `contiguous()` and the scatter behind `cat`."""
    assert src.shape == dst.shape and src.element_size() == dst.element_size() and 1 <= src.dim() <= 8
    nd = src.dim()
    arr = ctypes.c_longlong * nd
    rc = _fn("lt_strided_copy")(src.data_ptr(), dst.data_ptr(), nd, ctypes.cast(arr(*src.shape), c_void_p),
                                ctypes.cast(arr(*src.stride()), c_void_p), ctypes.cast(arr(*dst.stride()), c_void_p),
                                src.element_size(), _stream())
    _check(rc, "lt_strided_copy")
    return dst


def moe_expert_bwd(gu, dh_u, w, slot_src):
    """Pointwise part of the expert backward in one pass: gu [S, 2F], dh_u [S, F] bf16, gate weights w [S] fp32,
    slot_src [S, 2] int32 (first column < 0 marks a padding slot).  Returns (dgu [S, 2F], h * w [S, F], dw [S] fp32)."""
    S, F2 = gu.shape
    F = F2 // 2
    dgu = torch.empty_like(gu)
    hw = torch.empty((S, F), dtype=gu.dtype, device=gu.device)
    dw = torch.empty(S, dtype=torch.float32, device=gu.device)
    rc = _fn("lt_moe_expert_bwd")(gu.data_ptr(), dh_u.data_ptr(), w.data_ptr(), slot_src.data_ptr(), dgu.data_ptr(),
                                  hw.data_ptr(), dw.data_ptr(), S, F, _stream())
    _check(rc, "lt_moe_expert_bwd")
    return dgu, hw, dw
