"""Offline resharding of trainer checkpoints: a checkpoint written by one rank is cut for several layouts and put
together again bit for bit; gloo ranks that load a resharded checkpoint continue on the single-rank curve (weights and
AdamW moments are where the providers expect them); a checkpoint written by two ranks goes back to one; the Hugging Face
export of a checkpoint is loaded by `transformers`' own Llama with the same logits."""
import json
import os
import subprocess
import sys
import textwrap

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _single_rank_checkpoint(path, steps=2):
    from litetorch_b200.models.llama import LlamaConfig
    from litetorch_b200.trainer import Trainer
    cfg = LlamaConfig.tiny()
    tok = torch.randint(0, cfg.vocab_size, (2, 65), generator=torch.Generator().manual_seed(7))
    x, y = tok[:, :-1].contiguous(), tok[:, 1:].contiguous()
    tr = Trainer(cfg, seed=3, device="cpu", param_dtype=torch.float32, parallel="none")
    for _ in range(steps):
        tr.step(x, y)
    tr.save(path)
    return cfg, tr, x, y


def test_reshard_round_trips_bit_for_bit(tmp_path):
    from litetorch_b200 import checkpoint_tools as T
    src = str(tmp_path / "one")
    cfg, tr, x, y = _single_rank_checkpoint(src)
    _, meta, full = T.read_full_state(src)
    assert meta["step_count"] == 2 and meta["weights"] == "LocalWeights"
    for s in tr.engine.w.specs:
        assert torch.equal(full["master"][s.name], tr.engine.w.master_view(s.name))
    for world, tp, kind in ((2, 1, "ShardedWeights"), (2, 2, "HybridWeights"), (4, 2, "HybridWeights"), (2, 1, "HybridWeights")):
        mid = str(tmp_path / ("w%d_tp%d_%s" % (world, tp, kind)))
        out = T.reshard(src, mid, world, tp, weights=kind)
        assert sorted(f for f in os.listdir(out) if f.endswith(".ltw1")) == ["trainer.rank%05d.ltw1" % r for r in range(world)]
        back = str(tmp_path / ("back_" + os.path.basename(mid)))
        T.reshard(mid, back, 1)
        _, meta2, again = T.read_full_state(back)
        assert meta2["weights"] == "LocalWeights" and meta2["step_count"] == 2
        for q in T.QUANTITIES:
            for name, t in full[q].items():
                assert torch.equal(again[q][name], t), (world, tp, kind, q, name)
    with pytest.raises(T.CheckpointError):
        T.reshard(src, str(tmp_path / "bad"), 3, 2)
    r = subprocess.run([sys.executable, "-m", "litetorch_b200.checkpoint_tools", "info", "--src", src], capture_output=True,
                       text=True, timeout=120, cwd=ROOT)
    assert r.returncode == 0 and json.loads(r.stdout)["step_count"] == 2


WORKER = r'''
import json, os, sys, torch
sys.path.insert(0, %(root)r)
import torch.distributed as dist
from litetorch_b200.models.llama import LlamaConfig
from litetorch_b200.trainer import Trainer
rank = int(os.environ["RANK"])
dist.init_process_group("gloo", init_method="tcp://127.0.0.1:%%s" %% os.environ["MASTER_PORT"], rank=rank, world_size=int(os.environ["WORLD_SIZE"]))
torch.set_num_threads(2)
cfg = LlamaConfig.tiny()
tok = torch.randint(0, cfg.vocab_size, (2, 65), generator=torch.Generator().manual_seed(7))
x, y = tok[:, :-1].contiguous(), tok[:, 1:].contiguous()
tr = Trainer(cfg, seed=99, tp=2, device="cpu", param_dtype=torch.float32, parallel="hybrid")
tr.load(%(ckpt)r)
losses = [tr.step(x, y) for _ in range(2)]            # both ranks of the tensor-parallel pair see the same batch
tr.save(%(out)r)
if rank == 0:
    print("RESULT " + json.dumps({"losses": losses, "step": tr.engine.step_count}))
dist.barrier()
dist.destroy_process_group()
'''


def test_ranks_continue_from_a_resharded_checkpoint_and_back(tmp_path):
    from litetorch_b200 import checkpoint_tools as T
    from litetorch_b200.trainer import Trainer
    src = str(tmp_path / "one")
    cfg, tr, x, y = _single_rank_checkpoint(src)
    expected = [tr.step(x, y) for _ in range(2)]                       # the uninterrupted single-rank run
    two = str(tmp_path / "two")
    T.reshard(src, two, world=2, tp=2)
    script = tmp_path / "worker.py"
    script.write_text(WORKER % {"root": ROOT, "ckpt": two, "out": str(tmp_path / "two_later")})
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
                        "127.0.0.1", "--master-port", "29947", str(script)], capture_output=True, text=True, timeout=600,
                       env=dict(os.environ, OMP_NUM_THREADS="2"))
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    res = json.loads([l for l in r.stdout.splitlines() if l.startswith("RESULT ")][-1][7:])
    assert res["step"] == 4 and all(abs(a - b) < 2e-4 for a, b in zip(res["losses"], expected)), (res, expected)
    # what the two ranks saved goes back to one rank and matches the single-rank run after the same four steps
    one_again = str(tmp_path / "one_again")
    T.reshard(str(tmp_path / "two_later"), one_again, world=1)
    other = Trainer(cfg, seed=5, device="cpu", param_dtype=torch.float32, parallel="none")
    other.load(one_again)
    assert other.engine.step_count == 4
    diff = max(float((a - b).abs().max()) for a, b in zip(other.engine.w.parameters(), tr.engine.w.parameters()))
    assert diff < 1e-4 and abs(other.step(x, y) - tr.step(x, y)) < 2e-4


def test_export_hf_from_a_checkpoint(tmp_path):
    pytest.importorskip("transformers")
    pytest.importorskip("safetensors")
    from transformers import LlamaForCausalLM
    from litetorch_b200 import checkpoint_tools as T
    src = str(tmp_path / "one")
    cfg, tr, x, y = _single_rank_checkpoint(src)
    T.reshard(src, str(tmp_path / "four"), world=4, tp=2)
    T.export_hf(str(tmp_path / "four"), str(tmp_path / "hf"), dtype=torch.float32)
    hf = LlamaForCausalLM.from_pretrained(str(tmp_path / "hf"), torch_dtype=torch.float32).eval()
    with torch.no_grad():
        ref = hf(x).logits
    assert float((tr.engine.forward_logits(x) - ref).abs().max()) < 2e-4
