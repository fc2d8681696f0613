"""Crash and resume: a training process checkpoints (parameters LTW1, AdamW state LTAW, data position) and dies without
cleaning up; a fresh process loads the files and continues.  Its losses must equal those of an uninterrupted run."""
import json
import os
import subprocess
import sys

import pytest

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


def _bf16_run(steps, params, opt, data):
    import torch
    from litetorch_b200.core import _unwrap
    for x, y in data[:steps]:
        opt.zero_grad()
        w1, w2 = (_unwrap(p) for p in params)
        loss = ((torch.tanh(x.bfloat16() @ w1) @ w2).float() - y).pow(2).mean()
        loss.backward()
        opt.step()


def _bf16_setup(seed):
    import torch
    import litetorch_b200 as lt
    from litetorch_b200.core import Tensor
    g = torch.Generator().manual_seed(seed)
    params = [Tensor((torch.randn(16, 32, generator=g) * 0.3).bfloat16().requires_grad_(True)),
              Tensor((torch.randn(32, 4, generator=g) * 0.3).bfloat16().requires_grad_(True))]
    return params, lt.optim.AdamW(params, lr=1e-2, beta1=0.9, beta2=0.95, weight_decay=0.1)


def test_bf16_parameters_resume_exactly_in_either_load_order(tmp_path):
    """AdamW keeps fp32 masters of bf16 parameters; a checkpoint carries them, and a resumed run must neither write
    stale masters back over loaded weights nor lose the masters' low bits, whichever file is loaded first."""
    import torch
    import litetorch_b200 as lt
    from litetorch_b200.core import _unwrap
    g = torch.Generator().manual_seed(11)
    data = [(torch.randn(8, 16, generator=g), torch.randn(8, 4, generator=g)) for _ in range(6)]
    ref_p, ref_o = _bf16_setup(1)
    _bf16_run(6, ref_p, ref_o, data)
    p, o = _bf16_setup(1)
    _bf16_run(3, p, o, data)
    lt.save_parameters(p, str(tmp_path / "m.ltw"))
    lt.save(o, str(tmp_path / "o.bin"))
    for order in ("params_first", "optimizer_first"):
        q, qo = _bf16_setup(99)                       # another initialisation: everything must come from the files
        _bf16_run(1, q, qo, data[5:])                 # and the optimizer already holds (soon stale) masters
        if order == "params_first":
            lt.load_parameters(q, str(tmp_path / "m.ltw"))
            lt.load(qo, str(tmp_path / "o.bin"))
        else:
            lt.load(qo, str(tmp_path / "o.bin"))
            lt.load_parameters(q, str(tmp_path / "m.ltw"))
        _bf16_run(3, q, qo, data[3:])
        for a, b, ma, mb in zip(q, ref_p, qo.master, ref_o.master):
            assert torch.equal(_unwrap(a), _unwrap(b)), order
            assert torch.equal(ma, mb), order
    # a parameter overwritten by hand is taken over by the master instead of being reverted at the next step
    with torch.no_grad():
        _unwrap(p[0]).fill_(0.5)
    _bf16_run(1, p, o, data[3:])
    assert abs(float(_unwrap(p[0]).float().mean()) - 0.5) < 0.05


ZERO3_WORKER = r'''
import json, os, sys, torch
sys.path.insert(0, %(root)r)
import torch.distributed as dist
import litetorch_b200 as lt
from litetorch_b200.core import Tensor, _unwrap
from litetorch_b200.parallel.fsdp_api import FullyShardedDataParallel
from litetorch_b200.serialization import save_optimizer_sharded, load_optimizer_sharded, save_sharded, load_sharded
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo", init_method="tcp://127.0.0.1:%%s" %% os.environ["MASTER_PORT"], rank=rank, world_size=world)
ck = sys.argv[1]

def build(seed):
    torch.manual_seed(seed)
    m = lt.nn.Sequential([lt.nn.Linear(12, 10), lt.nn.Linear(10, 6)])
    f = FullyShardedDataParallel(m)
    o = lt.optim.ZeRO3Optimizer([p for p in m.parameters()], lr=1e-2, beta1=0.9, beta2=0.95, weight_decay=0.1)
    return m, f, o

def steps(f, o, m, n, start):
    out = []
    for s in range(start, start + n):
        g = torch.Generator().manual_seed(100 + s)
        x = torch.randn(4, 12, generator=g)
        f.gather_parameters()
        for p in m.parameters():
            _unwrap(p).grad = None
        y = _unwrap(f.forward(Tensor(x)))
        loss = y.pow(2).mean()
        loss.backward()
        f.shard_parameters()
        o.step()
        out.append(float(loss))
    return out

m, f, o = build(1)
full = steps(f, o, m, 6, 0)
m, f, o = build(1)
first = steps(f, o, m, 3, 0)
save_sharded(ck, [_unwrap(p.shard).detach() for p in m.parameters()], rank, world, tag="model")
save_optimizer_sharded(o, ck, rank, world)
dist.barrier()
m2, f2, o2 = build(5)
for p, t in zip(m2.parameters(), load_sharded(ck, rank, world, tag="model")):
    with torch.no_grad():
        _unwrap(p.shard).copy_(t.view_as(_unwrap(p.shard)))
load_optimizer_sharded(o2, ck, rank, world)
rest = steps(f2, o2, m2, 3, 3)
if rank == 0:
    print("RESULT " + json.dumps({"full": full, "first": first, "rest": rest, "step": o2.step_count}))
dist.barrier()
dist.destroy_process_group()
'''


def test_zero3_optimizer_sharded_save_and_load_on_two_ranks(tmp_path):
    script = str(tmp_path / "zero3_worker.py")
    with open(script, "w") as f:
        f.write(ZERO3_WORKER % {"root": ROOT})
    ck = str(tmp_path / "ck3")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", "29893", script, ck]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=dict(os.environ, OMP_NUM_THREADS="2"))
    assert r.returncode == 0, r.stdout[-1500:] + r.stderr[-3000:]
    res = json.loads([l for l in r.stdout.splitlines() if l.startswith("RESULT ")][-1][7:])
    assert res["first"] == res["full"][:3]
    assert all(abs(a - b) < 1e-6 for a, b in zip(res["rest"], res["full"][3:])), res
    assert res["step"] == 6


ELASTIC_WORKER = r'''
import json, os, sys, time, torch
sys.path.insert(0, %(root)r)
import torch.distributed as dist
from litetorch_b200.models.llama import LlamaConfig
from litetorch_b200.trainer import Trainer
from litetorch_b200.parallel import elastic
info = elastic.worker_info()
rank, world, attempt = info["rank"], info["world"], info["attempt"]
ck, mode = sys.argv[1], sys.argv[2]
torch.set_num_threads(2)
hb = elastic.start_heartbeat(0.1)
cfg = LlamaConfig.tiny()
B, T = 2, 64
gen = torch.Generator().manual_seed(7)
data = torch.randint(0, cfg.vocab_size, (6, world * B, T + 1), generator=gen)
tr = Trainer(cfg, seed=3, device="cpu", param_dtype=torch.float32, parallel="hybrid")
start = 0
if Trainer.latest_checkpoint(ck) is not None:
    tr.load(ck)
    start = tr.engine.step_count
losses = []
for s in range(start, 6):
    losses.append(tr.step(data[s, rank * B:(rank + 1) * B, :-1].contiguous(), data[s, rank * B:(rank + 1) * B, 1:].contiguous()))
    tr.save(ck)                                     # returns once the checkpoint of this step is complete and LATEST points at it
    if attempt == 0 and rank == 1 and s == 2:
        if mode == "exit":
            os._exit(17)                            # dies between steps, nothing in flight
        if mode == "hang":
            hb.stop()                               # stops beating and never joins the next collective
            time.sleep(600)
if rank == 0:
    print("RESULT " + json.dumps({"attempt": attempt, "start": start, "losses": losses}), flush=True)
if dist.is_initialized():                           # a group that shrank to one rank has no process group
    dist.barrier()
    dist.destroy_process_group()
'''


def _elastic_run(tmp, ck_name, mode, port):
    from litetorch_b200.parallel.elastic import ElasticLauncher
    script = os.path.join(tmp, "w.py")
    if not os.path.exists(script):
        with open(script, "w") as f:
            f.write(ELASTIC_WORKER % {"root": ROOT})
    env = dict(os.environ, OMP_NUM_THREADS="2")
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        env.pop(k, None)
    ck, logs = os.path.join(tmp, ck_name), os.path.join(tmp, "logs_" + ck_name)
    res = ElasticLauncher([sys.executable, script, ck, mode], nproc=2, max_restarts=2, base_port=port, heartbeat_ttl_s=2.0,
                          start_grace_s=120.0, env=env, log_dir=logs).run()
    out = []
    for a in range(len(res["attempts"])):
        with open(os.path.join(logs, "attempt%d_rank0.log" % a)) as f:
            out += [json.loads(l[7:]) for l in f.read().splitlines() if l.startswith("RESULT ")]
    return res, out


@pytest.fixture(scope="module")
def uninterrupted_run(tmp_path_factory):
    tmp = str(tmp_path_factory.mktemp("elastic_ref"))
    res, out = _elastic_run(tmp, "ck_ref", "none", 29640)
    assert res["ok"] and res["restarts"] == 0 and len(out) == 1 and len(out[0]["losses"]) == 6
    return out[0]["losses"]


@pytest.mark.parametrize("mode", ["exit", "hang"])
def test_elastic_launcher_restarts_the_group_and_the_run_ends_on_the_uninterrupted_curve(tmp_path, mode, uninterrupted_run):
    """Rank 1 dies (or stops beating and hangs) after the third step of the first attempt; the launcher stops the other rank,
    restarts both, they resume from the checkpoint and the last three losses equal those of a run nobody interrupted."""
    res, out = _elastic_run(str(tmp_path), "ck", mode, 29660 if mode == "exit" else 29700)
    assert res["ok"] and res["restarts"] == 1, res
    first = res["attempts"][0]
    assert ("exited with code 17" in first["reason"]) if mode == "exit" else ("heartbeats" in first["reason"]), first
    assert len(out) == 1 and out[0]["attempt"] == 1 and out[0]["start"] == 3
    assert all(abs(x - y) < 1e-6 for x, y in zip(out[0]["losses"], uninterrupted_run[3:])), (out, uninterrupted_run)


def test_elastic_launcher_shrinks_the_group_and_recuts_the_checkpoint(tmp_path):
    """A rank that fails every time at two ranks (a GPU lost for good): after one failed attempt the launcher halves the
    group, re-cuts the newest checkpoint for one rank, and the job resumes from step 3 and finishes there."""
    from litetorch_b200.parallel.elastic import ElasticLauncher
    script = tmp_path / "w.py"
    script.write_text((ELASTIC_WORKER % {"root": ROOT}).replace("if attempt == 0 and rank == 1 and s == 2:",
                                                                "if world == 2 and rank == 1 and s == 2:"))
    env = dict(os.environ, OMP_NUM_THREADS="2")
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        env.pop(k, None)
    ck, logs = str(tmp_path / "ck"), str(tmp_path / "logs")
    res = ElasticLauncher([sys.executable, str(script), ck, "exit"], nproc=2, max_restarts=2, base_port=29760, heartbeat_ttl_s=2.0,
                          start_grace_s=120.0, env=env, log_dir=logs, shrink_after=1, ckpt_dir=ck, tp=1).run()
    assert res["ok"] and res["restarts"] == 1 and res["nproc"] == 1, res
    assert [a["nproc"] for a in res["attempts"]] == [2, 1] and "code 17" in res["attempts"][0]["reason"]
    with open(os.path.join(logs, "attempt1_rank0.log")) as f:
        out = [json.loads(l[7:]) for l in f.read().splitlines() if l.startswith("RESULT ")]
    assert len(out) == 1 and out[0]["start"] == 3 and len(out[0]["losses"]) == 3
    assert os.path.isdir(ck + ".world2")                               # the two-rank cut is kept beside the new one
    with open(os.path.join(ck, open(os.path.join(ck, "LATEST")).read(), "trainer.manifest.json")) as f:
        meta = json.load(f)["meta"]
    assert meta["world_size"] == 1 and meta["weights"] == "LocalWeights" and meta["step_count"] == 6


def test_trainer_checkpoints_are_complete_or_absent(tmp_path):
    """`Trainer.save` builds a checkpoint in a temporary sub-directory and publishes it with two renames: what an interrupted
    save leaves behind is ignored by `load` and removed by the next save; only the newest `keep` checkpoints stay."""
    import torch
    from litetorch_b200.models.llama import LlamaConfig
    from litetorch_b200.serialization import CheckpointError
    from litetorch_b200.trainer import Trainer
    ck = str(tmp_path / "ck")
    cfg = LlamaConfig.tiny()
    tok = torch.randint(0, cfg.vocab_size, (2, 33), generator=torch.Generator().manual_seed(1))
    x, y = tok[:, :-1].contiguous(), tok[:, 1:].contiguous()
    tr = Trainer(cfg, seed=3, device="cpu", param_dtype=torch.float32, parallel="none")
    assert Trainer.latest_checkpoint(ck) is None
    with pytest.raises(CheckpointError):
        tr.load(ck)
    for _ in range(3):
        tr.step(x, y)
    tr.save(ck)
    assert open(os.path.join(ck, "LATEST")).read() == "step-00000003"
    # a save of step 4 that died after writing half a file
    os.makedirs(os.path.join(ck, ".step-00000004.tmp"))
    with open(os.path.join(ck, ".step-00000004.tmp", "trainer.rank00000.ltw1"), "wb") as f:
        f.write(b"LTW1\x05\x00")
    nxt = tr.step(x, y)
    other = Trainer(cfg, seed=9, device="cpu", param_dtype=torch.float32, parallel="none")
    other.load(ck)
    assert other.engine.step_count == 3 and abs(other.step(x, y) - nxt) < 1e-6
    for _ in range(2):
        tr.step(x, y)
        tr.save(ck)
    assert sorted(d for d in os.listdir(ck)) == ["LATEST", "step-00000005", "step-00000006"]


def test_background_save_holds_the_step_it_was_taken_at_and_is_published_later(tmp_path):
    """`save(..., background=True)` copies the state at once and writes it from a thread: steps taken meanwhile are not in
    the file, `LATEST` moves only when `finish_save` (or the next save / load) publishes it, and an error of the writer
    thread surfaces there."""
    import torch
    from litetorch_b200.models.llama import LlamaConfig
    from litetorch_b200.trainer import Trainer
    ck = str(tmp_path / "ck")
    cfg = LlamaConfig.tiny()
    tok = torch.randint(0, cfg.vocab_size, (2, 33), generator=torch.Generator().manual_seed(2))
    x, y = tok[:, :-1].contiguous(), tok[:, 1:].contiguous()
    tr = Trainer(cfg, seed=3, device="cpu", param_dtype=torch.float32, parallel="none")
    tr.step(x, y)
    tr.save(ck)                                             # step 1, published
    tr.step(x, y)
    tr.save(ck, background=True)                            # step 2, being written
    assert open(os.path.join(ck, "LATEST")).read() == "step-00000001"
    third = tr.step(x, y)                                   # training goes on; the file must not see this step
    tr.step(x, y)
    tr.finish_save()
    tr.finish_save()                                        # a no-op the second time
    assert open(os.path.join(ck, "LATEST")).read() == "step-00000002"
    other = Trainer(cfg, seed=9, device="cpu", param_dtype=torch.float32, parallel="none")
    other.load(ck)
    assert other.engine.step_count == 2 and abs(other.step(x, y) - third) < 1e-6
    # the next save publishes a pending one first; so does load
    tr.save(ck, background=True)                            # step 4
    tr.step(x, y)
    tr.save(ck, background=True)                            # step 5: step 4 is published before this one starts
    assert open(os.path.join(ck, "LATEST")).read() == "step-00000004"
    tr.load(ck)                                             # publishes step 5 and loads it
    assert tr.engine.step_count == 5
    # a writer that fails: the error is raised by finish_save and LATEST stays where it was
    import litetorch_b200.serialization as S
    real = S.save_sharded
    S.save_sharded = lambda *a, **k: (_ for _ in ()).throw(OSError("disk full"))
    try:
        tr.step(x, y)
        tr.save(ck, background=True)
        with pytest.raises(OSError, match="disk full"):
            tr.finish_save()
    finally:
        S.save_sharded = real
    assert open(os.path.join(ck, "LATEST")).read() == "step-00000005"


def test_trainer_checkpoint_carries_the_data_loader_position(tmp_path):
    """`Trainer.save(dir, loader=dl)` stores the loader's LTDL record (epoch, permutation, next index) with the tensors: a fresh
    trainer and a fresh loader built with the job's seed continue with the batches and the losses of the uninterrupted run, across
    the next reshuffle too."""
    import torch
    import litetorch_b200 as lt
    from litetorch_b200.core import _unwrap
    from litetorch_b200.models.llama import LlamaConfig
    from litetorch_b200.trainer import Trainer
    cfg = LlamaConfig.tiny()
    g = torch.Generator().manual_seed(5)
    toks = torch.randint(0, cfg.vocab_size, (24, 33), generator=g)

    def loader(seed):
        return lt.data.DataLoader(lt.data.TensorDataset(lt.Tensor(toks[:, :-1].float()), lt.Tensor(toks[:, 1:].float())), 4, True,
                                  lt.Device("cpu"), 2, seed=seed)

    def run(tr, dl, n):
        out = []
        for _ in range(n):
            b = dl.next()
            if b is None:
                dl.reset()
                b = dl.next()
            out.append(tr.step(_unwrap(b[0]).long(), _unwrap(b[1]).long()))
        return out

    make = lambda seed: Trainer(cfg, seed=seed, device="cpu", param_dtype=torch.float32, parallel="none")   # noqa: E731
    full = run(make(3), loader(1), 8)                       # crosses an epoch boundary (6 batches per epoch)
    tr, dl = make(3), loader(1)
    first = run(tr, dl, 4)
    ck = str(tmp_path / "ck")
    tr.save(ck, loader=dl)
    tr2, dl2 = make(9), loader(1)
    run(make(3), dl2, 2)                                    # the fresh loader is somewhere else before the load
    tr2.load(ck, loader=dl2)
    rest = run(tr2, dl2, 4)
    assert first == full[:4] and all(abs(a - b) < 1e-6 for a, b in zip(rest, full[4:])), (rest, full)


def test_lr_schedulers_drive_a_trainer():
    """`StepLR` / `CosineAnnealingLR` set `.lr` on whatever they are given: a Trainer exposes the engine's learning rate under that
    name, and the step really uses it (a run whose rate is cut to zero stops moving)."""
    import torch
    import litetorch_b200 as lt
    from litetorch_b200.models.llama import LlamaConfig
    from litetorch_b200.trainer import Trainer
    cfg = LlamaConfig.tiny()
    tok = torch.randint(0, cfg.vocab_size, (2, 33), generator=torch.Generator().manual_seed(4))
    x, y = tok[:, :-1].contiguous(), tok[:, 1:].contiguous()
    tr = Trainer(cfg, seed=3, lr=1e-3, device="cpu", param_dtype=torch.float32, parallel="none")
    sch = lt.optim.CosineAnnealingLR(tr, T_max=4, eta_min=0.0)
    rates = []
    for _ in range(4):
        tr.step(x, y)
        sch.step()
        rates.append(tr.get_lr())
    assert rates[0] < 1e-3 and rates == sorted(rates, reverse=True) and abs(rates[-1]) < 1e-12 and tr.engine.lr == rates[-1]
    frozen = [tr.step(x, y) for _ in range(3)]          # rate 0: the weights no longer change (weight decay is scaled by the rate too)
    assert abs(frozen[1] - frozen[2]) < 1e-7
    tr.set_lr(1e-3)
    moving = [tr.step(x, y) for _ in range(3)]
    assert moving[2] < moving[0] - 1e-4
