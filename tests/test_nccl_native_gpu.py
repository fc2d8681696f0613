"""NCCL through the native bridge, bootstrapped over the native TCP store, with no torch.distributed in the processes:
all-reduce, all-gather, reduce-scatter, broadcast and a send / receive pair on 2 GPUs (one child process per GPU)."""
import json
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r'''
import json, os, sys, torch
sys.path.insert(0, %(root)r)
rank, world, port = int(sys.argv[1]), int(sys.argv[2]), int(sys.argv[3])
torch.cuda.set_device(rank)
from litetorch_b200.parallel.process_group import TCPStore
from litetorch_b200.parallel.nccl_native import NativeNccl, nccl_version
store = TCPStore("127.0.0.1", port, is_server=(rank == 0), timeout_s=60.0)
comm = NativeNccl(store, rank, world)
dev = torch.device("cuda", rank)
out = {"version": nccl_version()}
a = torch.full((1 << 20,), float(rank + 1), device=dev, dtype=torch.bfloat16)
comm.all_reduce(a)
out["all_reduce"] = float(a.float().mean())
g = torch.empty(world * 1000, device=dev)
comm.all_gather(g, torch.full((1000,), float(rank), device=dev))
out["all_gather"] = [float(g[i * 1000]) for i in range(world)]
rs = torch.empty(512, device=dev)
comm.reduce_scatter(rs, torch.arange(world * 512, device=dev, dtype=torch.float32) * (rank + 1))
out["reduce_scatter"] = [float(rs[0]), float(rs[-1])]
b = torch.full((7,), float(rank), device=dev)
comm.broadcast(b, world - 1)
out["broadcast"] = float(b[3])
m = torch.arange(16, device=dev, dtype=torch.int32) + 100 * rank
r = torch.empty_like(m)
comm.group_start()
comm.send(m, (rank + 1) %% world)
comm.recv(r, (rank - 1) %% world)
comm.group_end()
torch.cuda.synchronize()
out["recv0"] = int(r[0])
store.barrier("done", world, timeout_s=60.0)
comm.destroy()
if rank == 0:
    print("RESULT " + json.dumps(out))
store.close() if rank != 0 else None
'''


def test_native_nccl_bridge_two_gpus(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    script = str(tmp_path / "nccl_worker.py")
    with open(script, "w") as f:
        f.write(WORKER % {"root": ROOT})
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    procs = [subprocess.Popen([sys.executable, script, str(r), "2", str(port)], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, env=env)
             for r in range(2)]
    outs = [p.communicate(timeout=300) for p in procs]
    assert all(p.returncode == 0 for p in procs), outs[0][1][-2000:] + outs[1][1][-2000:]
    res = json.loads([l for l in outs[0][0].splitlines() if l.startswith("RESULT ")][-1][7:])
    assert res["version"] >= 22000
    assert res["all_reduce"] == 3.0 and res["all_gather"] == [0.0, 1.0]
    assert res["reduce_scatter"] == [0.0, 511.0 * 3] and res["broadcast"] == 1.0 and res["recv0"] == 100
