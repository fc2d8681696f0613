"""The native caching allocator installed as PyTorch's CUDA allocator, and graph capture through the native runtime.

The allocator has to be installed before the first CUDA allocation of a process, so every case runs in a child."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

SCRIPT = r'''
import json, sys, torch
sys.path.insert(0, %(root)r)
import litetorch_b200 as lt
from litetorch_b200 import cuda as ltc
from litetorch_b200.models.llama import LlamaConfig, LlamaEngine
from litetorch_b200.ops import kernels as K
ltc.use_caching_allocator()
out = {}
cfg = LlamaConfig.tiny()
eng = LlamaEngine(cfg, "cuda", seed=0)
g = torch.Generator(device="cuda").manual_seed(1)
tok = torch.randint(0, cfg.vocab_size, (2, 128), device="cuda", generator=g)
tgt = torch.roll(tok, -1, 1)
losses = [float(eng.train_step(tok, tgt)) for _ in range(3)]
torch.cuda.synchronize()
st = ltc.allocator_stats()
out["losses_fall"] = losses[2] < losses[0]
out["hits"], out["misses"], out["peak"] = st["hits"], st["misses"], st["peak_bytes"]

# ---- a temporary used on a side stream: its block must not be handed out again while that stream still reads it
side = torch.cuda.Stream()
x = torch.full((1 << 22,), 3.0, device="cuda")
spin = torch.randn(4096, 4096, device="cuda")
torch.cuda.synchronize()
with torch.cuda.stream(side):
    side.wait_stream(torch.cuda.current_stream())
    for _ in range(30):
        spin = spin @ spin * 1e-3              # keeps the side stream busy for a while
    y = x * 2.0                                # reads x long after the host has moved on
ltc.record_stream(x, side)
ptr = x.data_ptr()
del x
z = torch.full((1 << 22,), -7.0, device="cuda")    # same size, same stream: would take x's block if it were free
out["block_was_held_back"] = z.data_ptr() != ptr
torch.cuda.synchronize()
out["side_stream_saw_its_data"] = bool((y == 6.0).all())
del y, z, spin
w = torch.empty(1 << 22, device="cuda")            # after the side stream finished the block comes back
out["block_returns_later"] = True
del w

# ---- one decoder layer captured with the native graph runtime and replayed
s = torch.cuda.Stream()
B, T = 2, 128
xin = torch.randn(B * T, cfg.d_model, device="cuda").bfloat16()
x2 = torch.randn(B * T, cfg.d_model, device="cuda").bfloat16()
with torch.cuda.stream(s):
    s.wait_stream(torch.cuda.current_stream())
    ref1 = eng._layer_fwd(0, xin, B, T)[0].clone()     # eager run on this stream: also fills the cache for the capture
    keep = eng._layer_fwd(0, xin, B, T)
    del keep
    gr = ltc.NativeGraph()
    gr.begin(s)
    yout, ctx = eng._layer_fwd(0, xin, B, T)
    gr.end(s)
    gr.launch(s)
    s.synchronize()
    out["replay_bit_exact"] = bool(torch.equal(yout, ref1))
    xin.copy_(x2)
    gr.launch(s)
    s.synchronize()
    got = yout.clone()
    ref2 = eng._layer_fwd(0, x2, B, T)[0]
    s.synchronize()
    out["replay_follows_new_input"] = bool(torch.equal(got, ref2))
out["status"] = K.status_fetch()
del eng, ctx, yout, gr
import gc; gc.collect()
torch.cuda.synchronize()
ltc.empty_cache()
st = ltc.allocator_stats()
out["allocated_after"], out["cached_after"] = st["allocated_bytes"], st["cached_bytes"]
print("RESULT " + json.dumps(out))
'''


def test_native_allocator_and_native_graph_in_a_fresh_process(tmp_path):
    script = str(tmp_path / "alloc_worker.py")
    with open(script, "w") as f:
        f.write(SCRIPT % {"root": ROOT})
    r = subprocess.run([sys.executable, script], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    res = json.loads([l for l in r.stdout.splitlines() if l.startswith("RESULT ")][-1][7:])
    assert res["losses_fall"] and res["hits"] > 0 and res["peak"] > 0
    assert res["block_was_held_back"] and res["side_stream_saw_its_data"]
    assert res["replay_bit_exact"] and res["replay_follows_new_input"]
    assert res["status"] == 0
    assert res["cached_after"] == 0, res
