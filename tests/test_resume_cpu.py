"""Crash and resume: a training process checkpoints (parameters LTW1, AdamW state LTAW, data position) and dies without
cleaning up; a fresh process loads the files and continues.  Its losses must equal those of an uninterrupted run."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r'''
import json, os, sys, torch
sys.path.insert(0, %(root)r)
import litetorch_b200 as lt
from litetorch_b200.core import Tensor
from litetorch_b200.models.gpt import GPT, GPTConfig
from litetorch_b200.ops import Ops
mode, ckdir = sys.argv[1], sys.argv[2]
cfg = GPTConfig()
B, T = 4, 32
torch.manual_seed(0)
data = torch.randint(0, cfg.vocab_size, (12, B, T + 1), generator=torch.Generator().manual_seed(7))
model = GPT(cfg, seed=3)
opt = lt.optim.AdamW(model.parameters(), lr=3e-3, beta1=0.9, beta2=0.95, weight_decay=0.1)
start = 0
if mode == "resume":
    lt.load_parameters(model, os.path.join(ckdir, "model.ltw"))
    lt.load(opt, os.path.join(ckdir, "optim.bin"))
    start = json.load(open(os.path.join(ckdir, "position.json")))["next_step"]
losses = []
for step in range(start, 6):
    seqs = data[step]
    tok, tgt = Tensor(seqs[:, :-1].float()), Tensor(seqs[:, 1:].reshape(-1).float())
    opt.zero_grad()
    loss = Ops.cross_entropy_loss(model(tok).view([B * T, cfg.vocab_size]), tgt)
    loss.backward()
    opt.step()
    losses.append(loss.item())
    if mode == "crash" and step == 2:
        lt.save_parameters(model, os.path.join(ckdir, "model.ltw"))
        lt.save(opt, os.path.join(ckdir, "optim.bin"))
        json.dump({"next_step": 3}, open(os.path.join(ckdir, "position.json"), "w"))
        print("LOSSES " + json.dumps(losses), flush=True)
        os._exit(17)                      # no interpreter shutdown, no destructors: a crash right after the checkpoint
print("LOSSES " + json.dumps(losses), flush=True)
'''


def _run(script, mode, ckdir, expect_rc):
    r = subprocess.run([sys.executable, script, mode, ckdir], capture_output=True, text=True, timeout=600,
                       env=dict(os.environ, OMP_NUM_THREADS="2"))
    assert r.returncode == expect_rc, r.stdout[-1500:] + r.stderr[-3000:]
    return json.loads([l for l in r.stdout.splitlines() if l.startswith("LOSSES ")][-1][7:])


def test_crash_after_checkpoint_then_resume_matches_uninterrupted_run(tmp_path):
    script = str(tmp_path / "worker.py")
    with open(script, "w") as f:
        f.write(WORKER % {"root": ROOT})
    ck = str(tmp_path / "ck")
    os.makedirs(ck)
    full = _run(script, "full", ck, 0)
    first = _run(script, "crash", ck, 17)
    rest = _run(script, "resume", ck, 0)
    assert len(full) == 6 and len(first) == 3 and len(rest) == 3
    assert first == full[:3]
    assert all(abs(a - b) < 1e-5 for a, b in zip(rest, full[3:])), (rest, full[3:])
    assert open(os.path.join(ck, "model.ltw"), "rb").read(4) == b"LTW1"
    # a checkpoint damaged after the crash is refused as a whole, before any parameter is touched
    blob = bytearray(open(os.path.join(ck, "model.ltw"), "rb").read())
    blob[len(blob) // 2] ^= 0x10
    open(os.path.join(ck, "model.ltw"), "wb").write(bytes(blob))
    r = subprocess.run([sys.executable, script, "resume", ck], capture_output=True, text=True, timeout=600)
    assert r.returncode != 0 and "CRC" in (r.stdout + r.stderr).upper()
