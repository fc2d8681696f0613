"""Context-parallel FlashAttention with in-kernel peer KV reads (forward) and peer Q/dO reads + remote dQ adds
(backward) against full attention computed on one device; 1 and 2 GPUs, contiguous and zigzag splits."""
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
import json, math, os, sys, torch
sys.path.insert(0, %(root)r)
import torch.distributed as dist
from litetorch_b200.ops import kernels as K
from litetorch_b200.parallel.cp import RingFlashContext, zigzag_split
local = int(os.environ["LOCAL_RANK"]); torch.cuda.set_device(local)
dist.init_process_group("nccl", device_id=torch.device("cuda", local))
rank, world = dist.get_rank(), dist.get_world_size()
dev = torch.device("cuda", local)
worst = 0.0
for (D, zig, causal, direct) in [(64, True, True, False), (128, True, True, False), (64, False, True, False),
                                (128, False, False, False), (64, True, True, True), (128, True, True, True)]:
    B, Hq, Hkv, Tl = 2, 4, 2, 512
    T = Tl * world
    g = torch.Generator(device="cpu").manual_seed(11)
    q, k, v, do = (torch.randn(B, T, h, D, generator=g) for h in (Hq, Hkv, Hkv, Hq))
    sp = (lambda t: zigzag_split(t, rank, world, 1)) if zig else (lambda t: t.chunk(world, 1)[rank].contiguous())
    ctx = RingFlashContext(B, Tl, Hq, Hkv, D, dev, zigzag=zig, direct_peer=direct)
    ql, kl, vl = (sp(t).to(dev).bfloat16().requires_grad_(True) for t in (q, k, v))
    for rep in range(2):
        for t in (ql, kl, vl): t.grad = None
        o = ctx.attention(ql, kl, vl, causal=causal)
        o.backward(sp(do).to(dev).bfloat16())
    # oracle: full attention in fp32 on this device
    qf, kf, vf = (t.to(dev).bfloat16().float().requires_grad_(True) for t in (q, k, v))
    G = Hq // Hkv
    s = torch.einsum("bthd,bshd->bhts", qf, kf.repeat_interleave(G, 2)) / math.sqrt(D)
    if causal:
        s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool, device=dev), 1), float("-inf"))
    of = torch.einsum("bhts,bshd->bthd", torch.softmax(s, -1), vf.repeat_interleave(G, 2))
    of.backward(do.to(dev).bfloat16().float())
    def rel(a, b): return float((a.float() - b).norm() / (b.norm() + 1e-9))
    errs = [rel(o, sp(of.detach())), rel(ql.grad, sp(qf.grad)), rel(kl.grad, sp(kf.grad)), rel(vl.grad, sp(vf.grad))]
    worst = max(worst, max(errs))
torch.cuda.synchronize()
from litetorch_b200.parallel.fsdp import check_symmetric_canaries
t = torch.tensor([worst, float(K.status_fetch()) + 1000.0 * check_symmetric_canaries()], device=dev); dist.all_reduce(t, op=dist.ReduceOp.MAX)
if rank == 0:
    print("RESULT " + json.dumps({"worst_rel_err": t[0].item(), "status": t[1].item()}))
dist.barrier(); dist.destroy_process_group()
'''


@pytest.mark.parametrize("nproc", [1, 2])
def test_cp_flash_matches_full_attention(nproc):
    if torch.cuda.device_count() < nproc:
        pytest.skip("needs %d GPUs" % nproc)
    script = os.path.join(tempfile.mkdtemp(prefix="lt_worker_"), "_cp_worker.py")
    with open(script, "w") as f:
        f.write(WORKER % {"root": ROOT})
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(nproc), "--master-addr",
           "127.0.0.1", "--master-port", "29751", script]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=dict(os.environ, NCCL_NVLS_ENABLE="0"))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    res = json.loads([l for l in r.stdout.splitlines() if l.startswith("RESULT ")][-1][7:])
    assert res["status"] == 0 and res["worst_rel_err"] < 2.5e-2, res
