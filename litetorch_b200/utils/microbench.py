"""Kernel micro-benchmarks: CUDA-event timing with an L2 flush between iterations.

    python -m litetorch_b200.utils.microbench gemm [--out FILE]
    python -m litetorch_b200.utils.microbench gemm8b       # one 8B layer's GEMMs, sustained, next to cuBLAS
    python -m litetorch_b200.utils.microbench fp8
    python -m litetorch_b200.utils.microbench attn
    python -m litetorch_b200.utils.microbench pointwise

Each line printed is a JSON object with the achieved TFLOP/s or GB/s and the fraction of the measured
peak (MEASURED_PEAKS.json at the repository root when present, else 1590 TFLOP/s / 6650 GB/s).
"""
from __future__ import annotations

import json
import os
import sys

import torch

_ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def peaks():
    p = os.path.join(_ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return {"tflops": float(d.get("bf16_tflops", 1590.0)), "gbs": float(d.get("hbm_gbs", 6650.0)), "src": "measured"}
    return {"tflops": 1590.0, "gbs": 6650.0, "src": "fallback"}


_flush = None


def flush_l2():
    global _flush
    if _flush is None:
        _flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    _flush.zero_()


def time_ms(fn, warmup=3, iters=10, flush=True):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        if flush:
            flush_l2()
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2]


def bench_gemm(out=None):
    from ..ops import kernels as K
    pk = peaks()
    shapes = [
        # (M, N, K, a_major, b_major, tag)   Llama-1.1B, 8192 tokens
        (8192, 2560, 2048, 0, 0, "qkv fwd"),
        (8192, 2048, 2048, 0, 0, "o fwd"),
        (8192, 11264, 2048, 0, 0, "gate_up fwd"),
        (8192, 2048, 5632, 0, 0, "down fwd"),
        (8192, 32000, 2048, 0, 0, "lm_head fwd"),
        (8192, 2048, 11264, 0, 1, "gate_up dgrad"),
        (8192, 5632, 2048, 0, 1, "down dgrad"),
        (11264, 2048, 8192, 1, 1, "gate_up wgrad"),
        (2048, 5632, 8192, 1, 1, "down wgrad"),
        (2560, 2048, 8192, 1, 1, "qkv wgrad"),
        (8192, 8192, 8192, 0, 0, "square"),
        (65536, 4096, 4096, 0, 0, "8B o fwd 64k tokens"),
    ]
    rows = []
    for M, N, Kd, am, bm, tag in shapes:
        a = torch.randn((M, Kd) if am == 0 else (Kd, M), device="cuda").bfloat16()
        b = torch.randn((N, Kd) if bm == 0 else (Kd, N), device="cuda").bfloat16()
        c = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        fl = 2.0 * M * N * Kd
        K.gemm_set_pair_mode(0)
        best = None
        for bn in (128, 256):
            ms = time_ms(lambda: K.gemm(a, b, a_major=am, b_major=bm, out=c, block_n=bn))
            if best is None or ms < best[0]:
                best = (ms, bn)
        K.gemm_set_pair_mode(2)
        ms_pair = time_ms(lambda: K.gemm(a, b, a_major=am, b_major=bm, out=c))
        K.gemm_set_tail_split(False)
        ms_pair_whole = time_ms(lambda: K.gemm(a, b, a_major=am, b_major=bm, out=c))
        K.gemm_set_tail_split(True)
        K.gemm_set_pair_mode(1)
        ms_auto = time_ms(lambda: K.gemm(a, b, a_major=am, b_major=bm, out=c))
        K.gemm_set_tail_split(False)
        K.gemm_set_pair_mode(0)
        ms_whole = time_ms(lambda: K.gemm(a, b, a_major=am, b_major=bm, out=c))
        K.gemm_set_pair_mode(1)
        K.gemm_set_tail_split(True)
        A = a if am == 0 else a.t()
        B = b.t() if bm == 0 else b
        ms_ref = time_ms(lambda: torch.matmul(A, B, out=c))
        K.check_status()
        row = {"kernel": "gemm_bf16", "tag": tag, "M": M, "N": N, "K": Kd, "a_major": am, "b_major": bm,
               "block_n": best[1], "ms": round(best[0], 4), "pair_ms": round(ms_pair, 4), "pair_no_tail_split_ms": round(ms_pair_whole, 4), "auto_ms": round(ms_auto, 4),
               "auto_tflops": round(fl / ms_auto / 1e9, 1),
               "auto_no_tail_split_ms": round(ms_whole, 4), "tflops": round(fl / best[0] / 1e9, 1),
               "frac_of_%s_peak" % pk["src"]: round(fl / best[0] / 1e9 / pk["tflops"], 3),
               "cublas_ms": round(ms_ref, 4), "cublas_tflops": round(fl / ms_ref / 1e9, 1)}
        rows.append(row)
        print(json.dumps(row), flush=True)
    if out:
        with open(out, "w") as f:
            for r in rows:
                f.write(json.dumps(r) + "\n")
    return rows


def bench_gemm_sustained(out=None):
    """The GEMMs of one Llama-3-8B layer (8192 tokens) timed the way they run inside a training step: each kernel
    back to back for about a second, so that the figure is taken at the clocks the 1 kW power cap allows, next to
    cuBLAS (torch.matmul) under the same load.  Operands are larger than L2 or nearly so; nothing is flushed."""
    from ..ops import kernels as K
    shapes = [
        (8192, 6144, 4096, 0, 0, "qkv fwd"), (8192, 4096, 4096, 0, 0, "o fwd"), (8192, 28672, 4096, 0, 0, "gate_up fwd"),
        (8192, 4096, 14336, 0, 0, "down fwd"), (8192, 4096, 28672, 0, 1, "gate_up dgrad"), (8192, 14336, 4096, 0, 1, "down dgrad"),
        (8192, 4096, 6144, 0, 1, "qkv dgrad"), (28672, 4096, 8192, 1, 1, "gate_up wgrad"), (4096, 14336, 8192, 1, 1, "down wgrad"),
        (6144, 4096, 8192, 1, 1, "qkv wgrad"),
    ]

    import threading
    try:
        import pynvml
        pynvml.nvmlInit()
        nv = pynvml.nvmlDeviceGetHandleByIndex(torch.cuda.current_device())
    except Exception:
        pynvml = nv = None

    def loop_ms(fn, seconds=1.2):
        """(ms per call, median SM MHz, median board W) over a loop of about `seconds`; clocks and power are read-only
        NVML queries made every 20 ms from a side thread once the loop has run for 0.3 s."""
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(); fn(); e1.record(); torch.cuda.synchronize()
        n = max(10, int(seconds * 1e3 / max(e0.elapsed_time(e1), 1e-3)))
        mhz, watts, stop = [], [], threading.Event()

        def sample():
            import time
            time.sleep(0.3)
            while not stop.is_set():
                try:
                    mhz.append(pynvml.nvmlDeviceGetClockInfo(nv, pynvml.NVML_CLOCK_SM))
                    watts.append(pynvml.nvmlDeviceGetPowerUsage(nv) / 1000.0)
                except Exception:
                    return
                time.sleep(0.02)

        th = threading.Thread(target=sample, daemon=True) if nv is not None else None
        if th:
            th.start()
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        stop.set()
        if th:
            th.join()
        med = lambda v: sorted(v)[len(v) // 2] if v else None
        return e0.elapsed_time(e1) / n, med(mhz), med(watts)

    rows = []
    for M, N, Kd, am, bm, tag in shapes:
        a = torch.randn((M, Kd) if am == 0 else (Kd, M), device="cuda").bfloat16()
        b = torch.randn((N, Kd) if bm == 0 else (Kd, N), device="cuda").bfloat16()
        c = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        A = a if am == 0 else a.t()
        B = b.t() if bm == 0 else b
        fl = 2.0 * M * N * Kd
        ms, mhz, w = loop_ms(lambda: K.gemm(a, b, a_major=am, b_major=bm, out=c))
        K.gemm_set_pair_mode(0)
        ms1, mhz1, w1 = loop_ms(lambda: K.gemm(a, b, a_major=am, b_major=bm, out=c))
        K.gemm_set_pair_mode(1)
        ms_ref, mhz_ref, w_ref = loop_ms(lambda: torch.matmul(A, B, out=c))
        K.check_status()
        row = {"kernel": "gemm_bf16 sustained", "tag": tag, "M": M, "N": N, "K": Kd, "ms": round(ms, 4), "tflops": round(fl / ms / 1e9, 1),
               "sm_mhz": mhz, "watts": w, "one_cta_ms": round(ms1, 4), "one_cta_tflops": round(fl / ms1 / 1e9, 1), "one_cta_sm_mhz": mhz1,
               "cublas_ms": round(ms_ref, 4), "cublas_tflops": round(fl / ms_ref / 1e9, 1), "cublas_sm_mhz": mhz_ref, "cublas_watts": w_ref,
               "ratio_to_cublas": round(ms_ref / ms, 3)}
        rows.append(row)
        print(json.dumps(row), flush=True)
    if out:
        with open(out, "w") as f:
            for r in rows:
                f.write(json.dumps(r) + "\n")
    return rows


def bench_fp8(out=None):
    """Block-scaled e4m3 GEMM (1x128 / 128x128 scales) and the row-scaled e4m3 GEMM against the bf16 kernel on the same shapes."""
    from ..ops import kernels as K
    pk = peaks()
    rows = []
    for M, N, Kd, tag in [(8192, 11264, 2048, "gate_up fwd"), (8192, 2048, 5632, "down fwd"), (8192, 8192, 8192, "square"),
                          (16384, 4096, 7168, "moe 671B-style expert width")]:
        x = torch.randn(M, Kd, device="cuda").bfloat16()
        w = (torch.randn(N, Kd, device="cuda") * 0.05).bfloat16()
        xq, xst = K.quant_fp8_1x128(x)
        wq = w.to(torch.float8_e4m3fn)
        ws = torch.ones((N + 127) // 128, Kd // 128, device="cuda")
        c = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        fl = 2.0 * M * N * Kd
        ms = time_ms(lambda: K.gemm_fp8_block(xq, xst, wq, ws, out=c, pairs=True))
        ms_one = time_ms(lambda: K.gemm_fp8_block(xq, xst, wq, ws, out=c, pairs=False))
        ms_q = time_ms(lambda: K.quant_fp8_1x128(x))
        ms_bf = time_ms(lambda: K.gemm(x, w, out=c))
        # the row-scaled kernel (one scale per token / channel, applied in the epilogue), burst and sustained
        rq, rs = K.quant_e4m3_rows(x)
        wq2, ws2 = K.quant_e4m3_rows(w)
        ms_rows = time_ms(lambda: K.gemm_e4m3(rq, rs, wq2, ws2, out=c))
        ms_rq = time_ms(lambda: K.quant_e4m3_rows(x))

        def sustained(fn, seconds=1.0):
            for _ in range(3):
                fn()
            n = max(10, int(seconds * 1e3 / max(ms_rows, 1e-3)))
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            for _ in range(n):
                fn()
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) / n

        y32 = K.gemm_e4m3(rq[:512], rs[:512], wq2, ws2, out_dtype=torch.float32)
        ref = (rq[:512].double() * rs[:512, None].double()) @ (wq2.double() * ws2[:, None].double()).t()
        acc_err = float((y32.double() - ref).norm() / ref.norm())      # accumulation error alone (same codes, float64)
        ms_rows_s = sustained(lambda: K.gemm_e4m3(rq, rs, wq2, ws2, out=c))
        ms_bf_s = sustained(lambda: K.gemm(x, w, out=c))
        K.check_status()
        row = {"kernel": "gemm_fp8_block", "tag": tag, "M": M, "N": N, "K": Kd, "ms": round(ms, 4),
               "tflops": round(fl / ms / 1e9, 1), "x_bf16_%s_peak" % pk["src"]: round(fl / ms / 1e9 / pk["tflops"], 3),
               "one_cta_ms": round(ms_one, 4), "quant_ms": round(ms_q, 4), "quant_gbs": round(M * Kd * 3 / ms_q / 1e6, 1),
               "bf16_kernel_ms": round(ms_bf, 4), "rows_ms": round(ms_rows, 4), "rows_tflops": round(fl / ms_rows / 1e9, 1),
               "rows_quant_ms": round(ms_rq, 4), "rows_sustained_tflops": round(fl / ms_rows_s / 1e9, 1),
               "bf16_sustained_tflops": round(fl / ms_bf_s / 1e9, 1), "rows_accumulation_rel_err": acc_err}
        rows.append(row)
        print(json.dumps(row), flush=True)
    if out:
        with open(out, "w") as f:
            for r_ in rows:
                f.write(json.dumps(r_) + "\n")
    return rows


def bench_attn(out=None):
    from ..ops import kernels as K
    pk = peaks()
    rows = []
    for (B, T, Hq, Hkv, D) in [(4, 2048, 32, 4, 64), (2, 8192, 32, 8, 128), (1, 32768, 12, 4, 128)]:
        q = torch.randn(B, T, Hq, D, device="cuda").bfloat16()
        k = torch.randn(B, T, Hkv, D, device="cuda").bfloat16()
        v = torch.randn(B, T, Hkv, D, device="cuda").bfloat16()
        do = torch.randn(B, T, Hq, D, device="cuda").bfloat16()
        fl = 4.0 * B * Hq * T * T * D / 2
        ms = time_ms(lambda: K.flash_fwd(q, k, v, causal=True))
        o, lse = K.flash_fwd(q, k, v, causal=True)
        row = {"kernel": "flash_fwd", "B": B, "T": T, "Hq": Hq, "Hkv": Hkv, "D": D, "ms": round(ms, 4),
               "tflops": round(fl / ms / 1e9, 1), "frac_of_%s_peak" % pk["src"]: round(fl / ms / 1e9 / pk["tflops"], 3)}
        qs, ks, vs = (x.transpose(1, 2) for x in (q, k, v))
        ms_ref = time_ms(lambda: torch.nn.functional.scaled_dot_product_attention(qs, ks, vs, is_causal=True, enable_gqa=True))
        row["sdpa_ms"] = round(ms_ref, 4)
        if K.has_kernel("lt_flash_bwd"):
            msb = time_ms(lambda: K.flash_bwd(q, k, v, o, lse, do, causal=True))
            row["bwd_ms"] = round(msb, 4)
            row["bwd_tflops"] = round(2.5 * fl / msb / 1e9, 1)
        K.check_status()
        rows.append(row)
        print(json.dumps(row), flush=True)
    if out:
        with open(out, "w") as f:
            for r in rows:
                f.write(json.dumps(r) + "\n")
    return rows


def bench_pointwise(out=None):
    from ..ops import kernels as K
    pk = peaks()
    rows = []
    M, D, F, V = 8192, 2048, 5632, 32000
    x = torch.randn(M, D, device="cuda").bfloat16()
    r = torch.randn(M, D, device="cuda").bfloat16()
    w = torch.ones(D, device="cuda").bfloat16()
    gu = torch.randn(M, 2 * F, device="cuda").bfloat16()
    dh = torch.randn(M, F, device="cuda").bfloat16()
    logits = torch.randn(M, V, device="cuda").bfloat16()
    tgt = torch.randint(0, V, (M,), device="cuda")
    n = 1 << 28
    p = torch.randn(n, device="cuda")
    g = torch.randn(n, device="cuda").bfloat16()
    m = torch.zeros(n, device="cuda")
    v = torch.zeros(n, device="cuda")
    p16 = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    y, s, mean, rstd = K.norm_fwd(x, w, None, r)
    stats = K.ce_stats(logits, tgt)
    cases = [
        ("rmsnorm_fwd(+res)", lambda: K.norm_fwd(x, w, None, r), M * D * 2 * 4),
        ("rmsnorm_bwd", lambda: K.norm_bwd(x, s, w, None, rstd), M * D * 2 * 3),
        ("swiglu_fwd", lambda: K.swiglu_fwd(gu), M * F * 2 * 3),
        ("swiglu_bwd", lambda: K.swiglu_bwd(gu, dh), M * F * 2 * 5),
        ("ce_stats", lambda: K.ce_stats(logits, tgt), M * V * 2),
        ("ce_finish", lambda: K.ce_finish(logits, tgt, stats), M * V * 2 * 2),
        ("adamw_flat", lambda: K.adam_flat(p, g, m, v, p16, lr=1e-4, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.1, step=1),
         n * (4 * 3 * 2 + 2 + 2)),
    ]
    for name, fn, nbytes in cases:
        ms = time_ms(fn)
        row = {"kernel": name, "ms": round(ms, 4), "GBps": round(nbytes / ms / 1e6, 1),
               "frac_of_%s_peak" % pk["src"]: round(nbytes / ms / 1e6 / pk["gbs"], 3)}
        rows.append(row)
        print(json.dumps(row), flush=True)
    K.check_status()
    if out:
        with open(out, "w") as f:
            for r_ in rows:
                f.write(json.dumps(r_) + "\n")
    return rows


if __name__ == "__main__":
    what = sys.argv[1] if len(sys.argv) > 1 else "gemm"
    out = sys.argv[sys.argv.index("--out") + 1] if "--out" in sys.argv else None
    {"gemm": bench_gemm, "gemm8b": bench_gemm_sustained, "fp8": bench_fp8, "attn": bench_attn, "pointwise": bench_pointwise}[what](out)
