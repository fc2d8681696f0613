"""Small, self-terminating workloads for `ncu` captures of one kernel each.

    python -m litetorch_b200.utils.profile_cases gemm|gemm_vs_cublas|gemm_wgrad|gemm_fp8|gemm_e4m3|gemm_rs|ag_gemm|rs_adamw|flash_fwd|flash_bwd|flash_fwd_d128|flash_bwd_d128|paged_decode|shard_gather|
                                                 rmsnorm|rmsnorm_bwd|swiglu|adamw|ce [reps]

Every case touches more than the 126 MB L2 but only a few hundred MB of device memory, launches the kernel a
handful of times and exits, so a capture with `-k regex:<kernel> -c 3` ends by itself in a minute or two.
"""
from __future__ import annotations

import sys

import torch


def main():
    from ..ops import kernels as K
    case = sys.argv[1] if len(sys.argv) > 1 else "gemm"
    reps = int(sys.argv[2]) if len(sys.argv) > 2 else 4
    dev = "cuda"
    torch.manual_seed(0)
    if case == "gemm":            # gate_up forward of the 1.1B model: 8192 x 11264 x 2048
        a = torch.randn(8192, 2048, device=dev).bfloat16()
        b = torch.randn(11264, 2048, device=dev).bfloat16()
        c = torch.empty(8192, 11264, device=dev, dtype=torch.bfloat16)
        fn = lambda: K.gemm(a, b, out=c)
    elif case == "gemm_vs_cublas":   # o-projection of the 8B model, once through this kernel and once through torch.matmul
        a = torch.randn(8192, 4096, device=dev).bfloat16()
        b = torch.randn(4096, 4096, device=dev).bfloat16()
        c = torch.empty(8192, 4096, device=dev, dtype=torch.bfloat16)
        fn = lambda: (K.gemm(a, b, out=c), torch.matmul(a, b.t(), out=c))
    elif case == "gemm_wgrad":    # down-projection weight gradient: 2048 x 5632 x 8192, both operands transposed
        a = torch.randn(8192, 2048, device=dev).bfloat16()
        b = torch.randn(8192, 5632, device=dev).bfloat16()
        c = torch.empty(2048, 5632, device=dev, dtype=torch.bfloat16)
        fn = lambda: K.gemm(a, b, a_major=1, b_major=1, out=c)
    elif case in ("flash_fwd", "flash_bwd"):
        B, T, Hq, Hkv, D = 4, 2048, 32, 4, 64
        q = torch.randn(B, T, Hq, D, device=dev).bfloat16()
        k = torch.randn(B, T, Hkv, D, device=dev).bfloat16()
        v = torch.randn(B, T, Hkv, D, device=dev).bfloat16()
        do = torch.randn(B, T, Hq, D, device=dev).bfloat16()
        o, lse = K.flash_fwd(q, k, v, causal=True)
        fn = (lambda: K.flash_fwd(q, k, v, causal=True)) if case == "flash_fwd" else (lambda: K.flash_bwd(q, k, v, o, lse, do, causal=True))
    elif case == "gemm_fp8":      # block-scaled e4m3 GEMM, gate_up forward shape
        x = torch.randn(8192, 2048, device=dev).bfloat16()
        w = (torch.randn(11264, 2048, device=dev) * 0.05).bfloat16()
        xq, xst = K.quant_fp8_1x128(x)
        wq, ws = K.quant_fp8_128x128(w)
        c = torch.empty(8192, 11264, device=dev, dtype=torch.bfloat16)
        fn = lambda: K.gemm_fp8_block(xq, xst, wq, ws, out=c)
    elif case == "gemm_e4m3":     # row-scaled e4m3 GEMM, gate_up forward shape
        x = torch.randn(8192, 2048, device=dev).bfloat16()
        w = (torch.randn(11264, 2048, device=dev) * 0.05).bfloat16()
        xq, xs = K.quant_e4m3_rows(x)
        wq, ws = K.quant_e4m3_rows(w)
        c = torch.empty(8192, 11264, device=dev, dtype=torch.bfloat16)
        fn = lambda: K.gemm_e4m3(xq, xs, wq, ws, out=c)
    elif case == "rmsnorm_bwd":
        x = torch.randn(65536, 2048, device=dev).bfloat16()
        dy = torch.randn(65536, 2048, device=dev).bfloat16()
        w = torch.ones(2048, device=dev).bfloat16()
        _, _, _, rstd = K.norm_fwd(x, w, None, None)
        fn = lambda: K.norm_bwd(dy, x, w, None, rstd)
    elif case == "rmsnorm":
        x = torch.randn(65536, 2048, device=dev).bfloat16()
        w = torch.ones(2048, device=dev).bfloat16()
        fn = lambda: K.norm_fwd(x, w, None, x)
    elif case == "swiglu":
        gu = torch.randn(16384, 11264, device=dev).bfloat16()
        fn = lambda: K.swiglu_fwd(gu)
    elif case == "adamw":
        n = 1 << 26
        p, m, v = torch.randn(n, device=dev), torch.zeros(n, device=dev), torch.zeros(n, device=dev)
        g = torch.randn(n, device=dev).bfloat16()
        p16 = torch.empty(n, device=dev, dtype=torch.bfloat16)
        fn = lambda: K.adam_flat(p, g, m, v, p16, lr=1e-4, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.1, step=1)
    elif case == "ce":
        logits = torch.randn(8192, 32000, device=dev).bfloat16()
        tgt = torch.randint(0, 32000, (8192,), device=dev)
        fn = lambda: K.ce_finish(logits, tgt, K.ce_stats(logits, tgt))
    elif case in ("flash_fwd_d128", "flash_bwd_d128"):      # the 8B shape: one sequence of 8192, 32 q / 8 kv heads of 128
        B, T, Hq, Hkv, D = 1, 8192, 32, 8, 128
        q = torch.randn(B, T, Hq, D, device=dev).bfloat16()
        k = torch.randn(B, T, Hkv, D, device=dev).bfloat16()
        v = torch.randn(B, T, Hkv, D, device=dev).bfloat16()
        do = torch.randn(B, T, Hq, D, device=dev).bfloat16()
        o, lse = K.flash_fwd(q, k, v, causal=True)
        fn = (lambda: K.flash_fwd(q, k, v, causal=True)) if case == "flash_fwd_d128" else (lambda: K.flash_bwd(q, k, v, o, lse, do, causal=True))
    elif case == "paged_decode":     # batch 32, 16 k context, 32 q / 4 kv heads of 64: 1 GB of K / V per launch
        S, H, Hkv, D, bs, ctx = 32, 32, 4, 64, 16, 16384
        nb = S * ctx // bs
        kc = torch.randn(nb, Hkv, bs, D, device=dev).bfloat16()
        vc = torch.randn(nb, Hkv, bs, D, device=dev).bfloat16()
        q = torch.randn(S, H, D, device=dev).bfloat16()
        bt = torch.arange(nb, device=dev, dtype=torch.int32).view(S, ctx // bs)
        cl = torch.full((S,), ctx, device=dev, dtype=torch.int32)
        fn = lambda: K.paged_decode(q, kc, vc, bt, cl, bs, 8, D ** -0.5)
    elif case == "shard_gather":     # 512 MB pulled from four "ranks" (local buffers stand in for peers)
        n = 1 << 26
        shards = [torch.randn(n, device=dev).bfloat16() for _ in range(4)]
        dst = torch.empty(4 * n, device=dev, dtype=torch.bfloat16)
        fn = lambda: K.gather_shards([s.data_ptr() for s in shards], [(0, n)], [dst], max_ctas=64)
    elif case in ("ag_gemm", "rs_adamw"):
        # the two ZeRO-3 kernels on a one-rank group: the gather CTAs copy the local shard while the GEMM CTAs wait on its flags
        # (ag_gemm), the reduce phase reads one "peer" (rs_adamw): everything but the NVLink hop
        import os
        import torch.distributed as dist
        from ..parallel.fsdp import SymmetricBuffer
        for k, v in (("RANK", "0"), ("WORLD_SIZE", "1"), ("MASTER_ADDR", "127.0.0.1"), ("MASTER_PORT", "29534")):
            os.environ.setdefault(k, v)
        torch.cuda.set_device(0)
        dist.init_process_group("nccl", device_id=torch.device("cuda", 0))
        if case == "ag_gemm":       # Llama-1.1B gate/up forward, the weight "gathered" by 8 gather CTAs
            Mt, N, Kd = 8192, 11264, 2048
            shard = SymmetricBuffer(N * Kd, torch.bfloat16, dev)
            shard.tensor.copy_((torch.randn(N * Kd, device=dev) * 0.02).bfloat16())
            full = torch.empty(N, Kd, device=dev, dtype=torch.bfloat16)
            gflags = torch.zeros(4096, dtype=torch.int32, device=dev)
            xt = torch.randn(Mt, Kd, device=dev).bfloat16()
            st = {"e": 0}

            def fn():
                st["e"] += 1
                K.ag_gemm(None, full, gather_operand=1, shard_ptrs=shard.ptrs, world=1, rank=0, rows_per_rank=N, flags=gflags,
                          epoch=st["e"], other=xt, n_comm=8)
        else:                       # one 64 M-element gradient bucket: bf16 gradients in, fp32 master / moments, bf16 parameters out
            n = 64 * 1024 * 1024
            grads = SymmetricBuffer(n, torch.bfloat16, dev)
            grads.tensor.copy_((torch.randn(n, device=dev) * 0.01).bfloat16())
            rs_flags = SymmetricBuffer(64 * 8, torch.int32, dev)
            master = torch.randn(n, device=dev)
            m1, v1 = torch.zeros(n, device=dev), torch.zeros(n, device=dev)
            p16 = torch.empty(n, device=dev, dtype=torch.bfloat16)
            st = {"e": 0}

            def fn():
                st["e"] += 1
                K.rs_adamw(grads.ptrs, None, master, m1, v1, p16, [(0, 0, n)], lr=1e-4, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.1,
                           step=st["e"], my_flags=rs_flags.tensor, peer_flag_ptrs=rs_flags.ptrs, slot=1, epoch=st["e"], world=1, rank=0)
    elif case == "gemm_rs":
        # GEMM -> reduce-scatter on a one-rank group: the scatter epilogue and the reduce phase without NVLink
        import os
        import torch.distributed as dist
        from ..parallel.tp_fused import TPFusedContext
        for k, v in (("RANK", "0"), ("WORLD_SIZE", "1"), ("MASTER_ADDR", "127.0.0.1"), ("MASTER_PORT", "29533")):
            os.environ.setdefault(k, v)
        torch.cuda.set_device(0)
        dist.init_process_group("nccl", device_id=torch.device("cuda", 0))
        tp = TPFusedContext(8192, 4096, dev)
        h = torch.randn(8192, 1792, device=dev).bfloat16()
        w_row = (torch.randn(4096, 1792, device=dev) * 0.02).bfloat16()
        fn = lambda: tp.gemm_scatter(h, w_row)
    else:
        raise SystemExit("unknown case " + case)
    for _ in range(reps):
        fn()
    torch.cuda.synchronize()
    K.check_status()
    print("ok", case)


if __name__ == "__main__":
    main()
