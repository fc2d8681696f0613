"""Fused all-gather->GEMM and GEMM->reduce-scatter (sequence-parallel TP) against the NCCL-collective path, 2 GPUs."""
import json
import os
import subprocess
import tempfile
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r'''
import json, os, sys, torch
sys.path.insert(0, %(root)r)
import torch.distributed as dist
import litetorch_b200 as lt
from litetorch_b200.core import _unwrap
from litetorch_b200.ops import kernels as K
from litetorch_b200.parallel.tp_fused import TPFusedContext, attach
local = int(os.environ["LOCAL_RANK"]); torch.cuda.set_device(local)
dist.init_process_group("nccl", device_id=torch.device("cuda", local))
rank, world = dist.get_rank(), dist.get_world_size()
dev = torch.device("cuda", local)
T, B, d, f = 512 * world, 2, 512, 1024
def build(fused):
    col = lt.nn.ColumnParallelLinear(d, f, True, gather_output=False, sequence_parallel=True).to(dev)
    row = lt.nn.RowParallelLinear(f, d, False, input_is_parallel=True, sequence_parallel=True).to(dev)
    for l in (col, row):
        l.weight = lt.Tensor(_unwrap(l.weight).detach().bfloat16().requires_grad_(True))
        if l.bias is not None: l.bias = lt.Tensor(_unwrap(l.bias).detach().bfloat16().requires_grad_(True))
    if fused:
        attach(TPFusedContext(T * B, max(d, f), dev), col, row)
    return col, row
g = torch.Generator(device="cpu").manual_seed(3)
x_full = torch.randn(T, B, d, generator=g)
res = {}
outs = {}
for fused in (False, True):
    col, row = build(fused)
    errs = []
    for it in range(3):                                  # several calls: slot parity, epochs, counters
        xs = (x_full * (1 + it)).chunk(world, 0)[rank].to(dev).bfloat16().requires_grad_(True)
        y = row(lt.Ops.gelu(col(lt.Tensor(xs))))
        yt = _unwrap(y)
        (yt.float() ** 2).sum().backward()
        outs[(fused, it)] = (yt.detach().float(), xs.grad.float(), _unwrap(col.weight).grad.float().clone(), _unwrap(row.weight).grad.float().clone())
        _unwrap(col.weight).grad = None; _unwrap(row.weight).grad = None
torch.cuda.synchronize()
def rel(a, b): return float((a - b).norm() / (b.norm() + 1e-9))
worst = 0.0
for it in range(3):
    for a, b in zip(outs[(True, it)], outs[(False, it)]):
        worst = max(worst, rel(a, b))
from litetorch_b200.parallel.fsdp import check_symmetric_canaries
t = torch.tensor([worst, float(K.status_fetch()) + 1000.0 * check_symmetric_canaries()], device=dev); dist.all_reduce(t, op=dist.ReduceOp.MAX)
if rank == 0:
    print("RESULT " + json.dumps({"worst_rel_err": t[0].item(), "status": t[1].item()}))
dist.barrier(); dist.destroy_process_group()
'''


@pytest.mark.parametrize("nproc", [1, 2])
def test_fused_tp_matches_nccl_path(nproc):
    if torch.cuda.device_count() < nproc:
        pytest.skip("needs %d GPUs" % nproc)
    script = os.path.join(tempfile.mkdtemp(prefix="lt_worker_"), "_tp_worker.py")
    with open(script, "w") as f:
        f.write(WORKER % {"root": ROOT})
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(nproc), "--master-addr",
           "127.0.0.1", "--master-port", "29741", script]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=dict(os.environ, NCCL_NVLS_ENABLE="0"))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    res = json.loads([l for l in r.stdout.splitlines() if l.startswith("RESULT ")][-1][7:])
    assert res["status"] == 0 and res["worst_rel_err"] < 3e-2, res


# Larger row counts: the gathered GEMM takes its tiles in groups of M blocks that start at the rank's own rows (a raster
# the small shapes above never reach), and the staging areas are poisoned so that a tile read before its rows landed,
# or a tile that was never computed, shows as NaN.
WORKER_LARGE = r'''
import json, os, sys, torch
sys.path.insert(0, %(root)r)
import torch.distributed as dist
from litetorch_b200.ops import kernels as K
from litetorch_b200.parallel.tp_fused import TPFusedContext, _ag_gemm_nn
local = int(os.environ["LOCAL_RANK"]); torch.cuda.set_device(local)
dist.init_process_group("nccl", device_id=torch.device("cuda", local))
rank, world = dist.get_rank(), dist.get_world_size()
dev = torch.device("cuda", local)
M, d = 8192, 1024
tp = TPFusedContext(M, d, dev)
for s in tp.stage: s.tensor.fill_(float("nan"))
tp.full.fill_(float("nan"))
torch.cuda.synchronize(); dist.barrier()
g = torch.Generator(device=dev).manual_seed(100 + rank)
def rel(a, b): return float((torch.nan_to_num(a.float(), nan=1e4) - b.float()).norm() / (b.float().norm() + 1e-9))
worst = 0.0
for it in range(3):
    for Kl, bm in ((1536, 0), (768, 1)):
        h = torch.randn(M, Kl, device=dev, generator=g).bfloat16()
        w = (torch.randn((d, Kl) if bm == 0 else (Kl, d), device=dev, generator=g) * 0.02).bfloat16()
        y = tp.gemm_scatter(h, w, b_major=bm)
        ref = torch.empty(M // world, d, device=dev)
        dist.reduce_scatter_tensor(ref, K.gemm(h, w, b_major=bm).float())
        worst = max(worst, rel(y, ref))
    for n_comm in (0, 8):
        tp.n_comm = n_comm
        xs = torch.randn(M // world, d, device=dev, generator=g).bfloat16()
        w = (torch.randn(1536, d, device=dev, generator=g) * 0.02).bfloat16()
        y, full = tp.gather_gemm(xs, w)
        parts = [torch.empty_like(xs) for _ in range(world)]
        dist.all_gather(parts, xs)
        xf = torch.cat(parts, 0)
        worst = max(worst, rel(y, K.gemm(xf, w)), rel(full, xf))
        dy = torch.randn(M // world, d, device=dev, generator=g).bfloat16()
        w2 = (torch.randn(d, 768, device=dev, generator=g) * 0.02).bfloat16()
        slot = tp.ag_calls & 1
        tp.ag_calls += 1
        tp.shard[slot].tensor[:dy.numel()].view_as(dy).copy_(dy)
        tp._barrier()
        dx = _ag_gemm_nn(tp, tp.full[:M * d].view(M, d), w2, slot, M // world)
        dist.all_gather(parts, dy)
        worst = max(worst, rel(dx, K.gemm(torch.cat(parts, 0), w2, b_major=1)))
torch.cuda.synchronize()
from litetorch_b200.parallel.fsdp import check_symmetric_canaries
t = torch.tensor([worst, float(K.status_fetch()) + 1000.0 * check_symmetric_canaries()], device=dev); dist.all_reduce(t, op=dist.ReduceOp.MAX)
if rank == 0:
    print("RESULT " + json.dumps({"worst_rel_err": t[0].item(), "status": t[1].item()}))
dist.barrier(); dist.destroy_process_group()
'''


@pytest.mark.parametrize("nproc", [1, 2])
def test_fused_tp_kernels_large_rows(nproc):
    if torch.cuda.device_count() < nproc:
        pytest.skip("needs %d GPUs" % nproc)
    script = os.path.join(tempfile.mkdtemp(prefix="lt_worker_"), "_tp_large_worker.py")
    with open(script, "w") as f:
        f.write(WORKER_LARGE % {"root": ROOT})
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(nproc), "--master-addr",
           "127.0.0.1", "--master-port", "29743", script]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=dict(os.environ, NCCL_NVLS_ENABLE="0"))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    res = json.loads([l for l in r.stdout.splitlines() if l.startswith("RESULT ")][-1][7:])
    assert res["status"] == 0 and res["worst_rel_err"] < 1e-2, res
