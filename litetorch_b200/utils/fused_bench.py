"""Achieved fraction of roofline of the fused compute + collective kernels (one JSON line per path, rank 0).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29500 \
        -m litetorch_b200.utils.fused_bench [--iters 10]

Roofline time of a fused path = the slower of (FLOPs / measured bf16 GEMM peak) and (bytes that must cross NVLink per
GPU / 770 GB/s, the measured peer-copy bandwidth per direction); fraction = roofline time / measured time.  Times are
CUDA events on the launching stream, maximum over ranks, after warm-up, with the operands re-published every
iteration as the training step does.  Also printed: the same GEMM without any communication (the compute floor on
this kernel) and the unfused pair (NCCL collective + GEMM) for comparison.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from .microbench import peaks

NVLINK_GBS = 770.0


def _time(fn, iters, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from ..ops import kernels as K
    from ..parallel.fsdp import SymmetricBuffer
    from ..parallel.tp_fused import TPFusedContext
    dev = torch.device("cuda", local)
    pk = peaks()
    peak_flops = pk["tflops"] * 1e12
    W = world
    out = []

    def report(name, ms, flops, nvlink_bytes, extra):
        t_c = flops / peak_flops * 1e3
        t_n = nvlink_bytes / (NVLINK_GBS * 1e9) * 1e3
        roof = max(t_c, t_n)
        row = {"path": name, "n_gpus": W, "ms": round(ms, 4), "roofline_ms": round(roof, 4),
               "bound": "compute" if t_c >= t_n else "nvlink", "fraction_of_roofline": round(roof / ms, 3),
               "peak_source": pk["src"]}
        row.update(extra)
        out.append(row)
        if rank == 0:
            print(json.dumps(row), flush=True)

    # ---------------------------------------------------------------- TP / SP: all-gather -> GEMM and GEMM -> reduce-scatter
    # Llama-3-8B widths at 8192 tokens per tensor-parallel group: gate/up column slice and down-projection row slice.
    M, d, F = 8192, 4096, 14336
    Fl = max(256, (2 * F // W) // 256 * 256)          # local gate|up columns
    Kl = max(256, (F // W) // 256 * 256)              # local down-projection input features
    tp = TPFusedContext(M, d, dev, n_comm=8)
    x_shard = torch.randn(M // W, d, device=dev).bfloat16()
    w_col = (torch.randn(Fl, d, device=dev) * 0.02).bfloat16()
    ms = _time(lambda: tp.gather_gemm(x_shard, w_col), args.iters)
    x_full = torch.randn(M, d, device=dev).bfloat16()
    ms_local = _time(lambda: K.gemm(x_full, w_col), args.iters)

    def unfused_ag():
        parts = [torch.empty_like(x_shard) for _ in range(W)]
        dist.all_gather(parts, x_shard)
        K.gemm(torch.cat(parts, 0), w_col)
    ms_nccl = _time(unfused_ag, args.iters)
    report("tp all-gather -> GEMM (ag_gemm, A gathered)", ms, 2.0 * M * Fl * d, (W - 1) / W * M * d * 2,
           {"shape": [M, Fl, d], "gemm_only_ms": round(ms_local, 4), "nccl_then_gemm_ms": round(ms_nccl, 4)})

    h = torch.randn(M, Kl, device=dev).bfloat16()
    w_row = (torch.randn(d, Kl, device=dev) * 0.02).bfloat16()
    ms = _time(lambda: tp.gemm_scatter(h, w_row), args.iters)
    ms_local = _time(lambda: K.gemm(h, w_row), args.iters)

    def unfused_rs():
        y = K.gemm(h, w_row)
        o = torch.empty(M // W, d, device=dev, dtype=torch.bfloat16)
        dist.reduce_scatter_tensor(o, y)
    ms_nccl = _time(unfused_rs, args.iters)
    report("tp GEMM -> reduce-scatter (gemm_rs)", ms, 2.0 * M * d * Kl, (W - 1) / W * M * d * 2,
           {"shape": [M, d, Kl], "gemm_only_ms": round(ms_local, 4), "gemm_then_nccl_ms": round(ms_nccl, 4)})

    # ---------------------------------------------------------------- ZeRO-3: weight all-gather -> GEMM (B gathered by N blocks)
    # Llama-1.1B gate/up forward: 8192 tokens x [11264, 2048] weight sharded by rows over the ranks.
    Mt, N, Kd = 8192, 11264, 2048
    rows = N // W // 256 * 256
    Nw = rows * W
    shard = SymmetricBuffer(rows * Kd, torch.bfloat16, dev)
    shard.tensor.copy_((torch.randn(rows * Kd, device=dev) * 0.02).bfloat16())
    flags_sym = SymmetricBuffer(64 * 8, torch.int32, dev)
    full = torch.empty(Nw, Kd, device=dev, dtype=torch.bfloat16)
    gflags = torch.zeros(4096, dtype=torch.int32, device=dev)
    xt = torch.randn(Mt, Kd, device=dev).bfloat16()
    state = {"e": 0, "b": 0}

    def fsdp_ag():
        state["b"] += 1
        K.signal_barrier(flags_sym.tensor, flags_sym.ptrs, 0, state["b"], W, rank)
        state["e"] += 1
        K.ag_gemm(None, full, gather_operand=1, shard_ptrs=shard.ptrs, world=W, rank=rank, rows_per_rank=rows, flags=gflags,
                  epoch=state["e"], other=xt, n_comm=8)
    try:
        ms = _time(fsdp_ag, args.iters)
        w_local = torch.randn(Nw, Kd, device=dev).bfloat16()
        ms_local = _time(lambda: K.gemm(xt, w_local), args.iters)
        report("zero-3 weight all-gather -> GEMM (ag_gemm, B gathered)", ms, 2.0 * Mt * Nw * Kd, (W - 1) / W * Nw * Kd * 2,
               {"shape": [Mt, Nw, Kd], "gemm_only_ms": round(ms_local, 4)})
    except Exception as e:   # the wrapper's keyword set differs between operand kinds; report instead of failing the run
        if rank == 0:
            print(json.dumps({"path": "zero-3 weight all-gather -> GEMM", "error": str(e)[:200]}), flush=True)

    # ---------------------------------------------------------------- ZeRO-3: reduce-scatter -> AdamW
    n = 64 * 1024 * 1024 // W * W          # gradient elements of one bucket (bf16), n / W updated per rank
    grads = SymmetricBuffer(n, torch.bfloat16, dev)
    grads.tensor.copy_((torch.randn(n, device=dev) * 0.01).bfloat16())
    rs_flags = SymmetricBuffer(64 * 8, torch.int32, dev)
    per = n // W
    master = torch.randn(per, device=dev)
    m1, v1 = torch.zeros(per, device=dev), torch.zeros(per, device=dev)
    p16 = torch.empty(per, device=dev, dtype=torch.bfloat16)
    st = {"e": 0}

    def rs():
        st["e"] += 1
        K.rs_adamw(grads.ptrs, None, master, m1, v1, p16, [(rank * per, 0, per)], lr=1e-4, beta1=0.9, beta2=0.95, eps=1e-8,
                   wd=0.1, step=st["e"], my_flags=rs_flags.tensor, peer_flag_ptrs=rs_flags.ptrs, slot=1, epoch=st["e"],
                   world=W, rank=rank)
    ms = _time(rs, args.iters)
    # no FLOP bound here: the two floors are peer reads over NVLink and the local AdamW traffic over HBM
    t_n = (W - 1) * per * 2 / (NVLINK_GBS * 1e9) * 1e3
    t_h = per * (2 + 4 * 3 * 2 + 2) / (pk["gbs"] * 1e9) * 1e3
    roof = max(t_n, t_h)
    row = {"path": "zero-3 reduce-scatter -> AdamW (rs_adamw)", "n_gpus": W, "ms": round(ms, 4), "roofline_ms": round(roof, 4),
           "bound": "nvlink" if t_n >= t_h else "hbm", "fraction_of_roofline": round(roof / ms, 3), "elements_per_rank": per,
           "peak_source": pk["src"]}
    if rank == 0:
        print(json.dumps(row), flush=True)
    status = K.status_fetch()
    if rank == 0:
        print(json.dumps({"device_status": status}), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
