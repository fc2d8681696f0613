"""Expert-parallel MoE with dispatch/combine fused into the grouped GEMMs against the all-to-all implementation."""
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
from litetorch_b200.parallel.ep import MoEFeedForward
from litetorch_b200.parallel.ep_fused import MoEFusedFeedForward
local = int(os.environ["LOCAL_RANK"]); torch.cuda.set_device(local)
dist.init_process_group("nccl", device_id=torch.device("cuda", local))
rank, world = dist.get_rank(), dist.get_world_size()
dev = torch.device("cuda", local)
d, F, E, k, N = 256, 512, 4, 2, 640
ref = MoEFeedForward(d, F, E, k, capacity_factor=1.25, group=dist.group.WORLD, dtype=torch.bfloat16, device=dev, seed=5)
fus = MoEFusedFeedForward(d, F, E, k, capacity_factor=1.25, group=dist.group.WORLD, device=dev, seed=5, max_tokens=1024)
worst = 0.0
def rel(a, b): return float((a.float() - b.float()).norm() / (b.float().norm() + 1e-9))
for it in range(3):
    g = torch.Generator(device="cpu").manual_seed(100 + 10 * it + rank)
    x = torch.randn(N, d, generator=g)
    dy = torch.randn(N, d, generator=g).to(dev).bfloat16()
    outs = []
    for m in (ref, fus):
        for p in m.parameters(): p.zero_grad()
        xi = x.to(dev).bfloat16().requires_grad_(True)
        y = _unwrap(m(lt.Tensor(xi)))
        y.backward(dy)
        outs.append((y.detach(), xi.grad, _unwrap(m.w_gate_up).grad.clone(), _unwrap(m.w_down).grad.clone(), _unwrap(m.gate_weight).grad.clone()))
    worst = max([worst] + [rel(a, b) for a, b in zip(outs[1], outs[0])])
    assert fus.last_dropped == ref.last_dropped
torch.cuda.synchronize()
from litetorch_b200.parallel.fsdp import check_symmetric_canaries
t = torch.tensor([worst, float(K.status_fetch()) + 1000.0 * check_symmetric_canaries()], device=dev); dist.all_reduce(t, op=dist.ReduceOp.MAX)
if rank == 0:
    print("RESULT " + json.dumps({"worst_rel_err": t[0].item(), "status": t[1].item(), "dropped": fus.last_dropped}))
dist.barrier(); dist.destroy_process_group()
'''


@pytest.mark.parametrize("nproc", [1, 2])
def test_fused_moe_matches_all_to_all_path(nproc):
    if torch.cuda.device_count() < nproc:
        pytest.skip("needs %d GPUs" % nproc)
    script = os.path.join(tempfile.mkdtemp(prefix="lt_worker_"), "_moe_worker.py")
    with open(script, "w") as f:
        f.write(WORKER % {"root": ROOT})
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(nproc), "--master-addr",
           "127.0.0.1", "--master-port", "29761", script]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=dict(os.environ, NCCL_NVLS_ENABLE="0"))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    res = json.loads([l for l in r.stdout.splitlines() if l.startswith("RESULT ")][-1][7:])
    assert res["status"] == 0 and res["worst_rel_err"] < 3e-2, res
