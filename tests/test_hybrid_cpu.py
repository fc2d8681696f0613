"""FSDP x TP (+ sequence parallel) schedule of the Llama engine on gloo ranks against the single-rank engine.

The "collective" back-end of `HybridWeights` runs the same forward/backward schedule, tensor-parallel slicing, ZeRO-3
shard layout and per-bucket optimizer updates as the fused CUDA back-end, on torch.distributed collectives; here it is
compared in fp32 with `LocalWeights` on the whole batch: loss, every gradient, and the parameters after AdamW steps."""
import json
import os
import subprocess
import sys
import textwrap

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r'''
import json, os, sys, torch
sys.path.insert(0, %(root)r)
import torch.distributed as dist
from litetorch_b200.models.llama import LlamaConfig, LlamaEngine, LocalWeights
from litetorch_b200.parallel.hybrid import HybridWeights
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo", init_method="tcp://127.0.0.1:%%s" %% os.environ["MASTER_PORT"], rank=rank, world_size=world)
torch.set_num_threads(2)
tp, ckpt = %(tp)d, %(ckpt)s
dp = world // tp
cfg = LlamaConfig.tiny()
B, T = 2, 64
gen = torch.Generator().manual_seed(7)
tok_all = torch.randint(0, cfg.vocab_size, (dp * B, T + 1), generator=gen)
w = HybridWeights(cfg, "cpu", tp=tp, seed=3, param_dtype=torch.float32)
eng = LlamaEngine(cfg, "cpu", weights=w, activation_checkpointing=ckpt, world_size=dp)
d = rank // tp
tok, tgt = tok_all[d * B:(d + 1) * B, :-1], tok_all[d * B:(d + 1) * B, 1:]
# reference: the whole batch on one rank
wr = LocalWeights(cfg, "cpu", seed=3, param_dtype=torch.float32)
ref = LlamaEngine(cfg, "cpu", weights=wr, activation_checkpointing=False)
p0 = max(float((a - b).abs().max()) for a, b in zip(w.parameters(), wr.parameters()))
loss = eng.forward_backward(tok, tgt)
lt = torch.tensor([float(loss)])
dist.all_reduce(lt)
loss_ref = float(ref.forward_backward(tok_all[:, :-1], tok_all[:, 1:]))
gerr = 0.0
for s in w.specs:
    g = w.gather_full_grad(s.name)
    gr = wr.g(s.name).float()
    gerr = max(gerr, float((g - gr).abs().max()) / (float(gr.abs().max()) + 1e-12))
losses, losses_ref = [], []
for it in range(3):
    l = eng.train_step(tok, tgt)
    lt2 = torch.tensor([float(l)]); dist.all_reduce(lt2)
    losses.append(float(lt2) / world)
    losses_ref.append(float(ref.train_step(tok_all[:, :-1], tok_all[:, 1:])))
perr = max(float((a - b).abs().max()) for a, b in zip(w.parameters(), wr.parameters()))
ev = torch.tensor([float(eng.eval_loss(tok, tgt))]); dist.all_reduce(ev)
ev_ref = float(ref.eval_loss(tok_all[:, :-1], tok_all[:, 1:]))
assert abs(float(ev) / world - ev_ref) < 2e-4, (float(ev) / world, ev_ref)
if rank == 0:
    print("RESULT " + json.dumps(dict(p0=p0, loss=float(lt) / world, loss_ref=loss_ref, gerr=gerr, losses=losses,
                                      losses_ref=losses_ref, perr=perr, trace=w._trace_done)))
dist.barrier()
dist.destroy_process_group()
'''


def _run(tmp_path, nproc, tp, ckpt, port):
    script = os.path.join(str(tmp_path), "hybrid_worker.py")
    with open(script, "w") as f:
        f.write(WORKER % {"root": ROOT, "tp": tp, "ckpt": ckpt})
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(nproc), "--master-addr",
           "127.0.0.1", "--master-port", str(port), script]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=dict(os.environ, OMP_NUM_THREADS="2"))
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    return json.loads([l for l in r.stdout.splitlines() if l.startswith("RESULT ")][-1][7:])


@pytest.mark.parametrize("nproc,tp,ckpt", [(4, 2, True), (2, 2, False), (2, 1, False)])
def test_hybrid_matches_single_rank(tmp_path, nproc, tp, ckpt):
    res = _run(tmp_path, nproc, tp, ckpt, 29871 + nproc * 3 + tp)
    assert res["p0"] == 0.0                                  # same initial model under every layout
    assert abs(res["loss"] - res["loss_ref"]) < 1e-5
    assert res["gerr"] < 1e-4
    for a, b in zip(res["losses"], res["losses_ref"]):
        assert abs(a - b) < 1e-4
    assert res["perr"] < 1e-4
    if nproc // tp > 1:
        assert res["trace"]                                  # the prefetch schedule was recorded after the first full step


RESUME_WORKER = r'''
import json, os, sys, torch
sys.path.insert(0, %(root)r)
import torch.distributed as dist
from litetorch_b200.models.llama import LlamaConfig
from litetorch_b200.trainer import Trainer
from litetorch_b200.serialization import CheckpointError
rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
tp, ck = %(tp)d, sys.argv[1]
torch.set_num_threads(2)
cfg = LlamaConfig.tiny()
B, T = 2, 64
dp = world // tp
gen = torch.Generator().manual_seed(7)
data = torch.randint(0, cfg.vocab_size, (6, dp * B, T + 1), generator=gen)
def batch(s):
    d = rank // tp
    return data[s, d * B:(d + 1) * B, :-1].contiguous(), data[s, d * B:(d + 1) * B, 1:].contiguous()
def make(seed):
    return Trainer(cfg, seed=seed, tp=tp, device="cpu", param_dtype=torch.float32, parallel="hybrid" if world > 1 else "none")
a = make(3)
full = [a.step(*batch(s)) for s in range(6)]
b = make(3)
first = [b.step(*batch(s)) for s in range(3)]
b.save(ck)
c = make(11)                     # other weights, fresh optimizer: everything must come from the checkpoint
c.step(*batch(5))
c.load(ck)
rest = [c.step(*batch(s)) for s in range(3, 6)]
refused = False
try:
    import dataclasses
    other = Trainer(dataclasses.replace(LlamaConfig.tiny(), ffn=1024), seed=3, tp=tp, device="cpu", param_dtype=torch.float32,
                    parallel="hybrid" if world > 1 else "none")
    other.load(ck)
except CheckpointError:
    refused = True
if rank == 0:
    print("RESULT " + json.dumps({"full": full, "first": first, "rest": rest, "refused": refused, "step": c.engine.step_count}))
if world > 1:
    dist.barrier()
    dist.destroy_process_group()
'''


@pytest.mark.parametrize("nproc,tp", [(1, 1), (4, 2)])
def test_trainer_save_load_resumes_on_the_same_curve(tmp_path, nproc, tp):
    script = os.path.join(str(tmp_path), "resume_worker.py")
    with open(script, "w") as f:
        f.write(RESUME_WORKER % {"root": ROOT, "tp": tp})
    ck = os.path.join(str(tmp_path), "ck")
    if nproc == 1:
        cmd = [sys.executable, script, ck]
    else:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(nproc), "--master-addr",
               "127.0.0.1", "--master-port", "29877", script, ck]
    env = dict(os.environ, OMP_NUM_THREADS="2")
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        env.pop(k, None)
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    res = json.loads([l for l in r.stdout.splitlines() if l.startswith("RESULT ")][-1][7:])
    assert res["first"] == res["full"][:3]
    assert all(abs(x - y) < 1e-6 for x, y in zip(res["rest"], res["full"][3:])), res
    assert res["refused"] and res["step"] == 6


CONFIG_WORKER = r'''
import json, os, sys, torch
sys.path.insert(0, %(root)r)
import torch.distributed as dist
import litetorch_b200 as lt
from litetorch_b200.trainer import Trainer
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
run = lt.config.load("llama3-8b-fsdp-tp2")          # tensor parallelism 2 x ZeRO-3, shrunk to a toy model by overrides
run = lt.config.apply_env(run, {"LT_CFG_MODEL__VOCAB": "512", "LT_CFG_MODEL__N_LAYERS": "2", "LT_CFG_MODEL__D_MODEL": "256",
                                "LT_CFG_MODEL__N_Q": "4", "LT_CFG_MODEL__N_KV": "2", "LT_CFG_MODEL__HEAD_DIM": "64",
                                "LT_CFG_MODEL__FFN": "512", "LT_CFG_SEQ_LEN": "64"})
tr = Trainer.from_config(run, device="cpu", param_dtype=torch.float32)
g = torch.Generator().manual_seed(rank // tr.tp)
tok = torch.randint(0, 512, (2, 65), generator=g)
losses = [tr.step(tok[:, :-1].contiguous(), tok[:, 1:].contiguous()) for _ in range(3)]
if rank == 0:
    print("RESULT " + json.dumps({"tp": tr.tp, "dp": tr.dp, "weights": type(tr.engine.w).__name__, "losses": losses}))
dist.barrier()
dist.destroy_process_group()
'''


def test_trainer_from_config_builds_the_fsdp_tp_layout(tmp_path):
    script = os.path.join(str(tmp_path), "config_worker.py")
    with open(script, "w") as f:
        f.write(CONFIG_WORKER % {"root": ROOT})
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "4", "--master-addr", "127.0.0.1",
           "--master-port", "29879", script]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=dict(os.environ, OMP_NUM_THREADS="2"))
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    res = json.loads([l for l in r.stdout.splitlines() if l.startswith("RESULT ")][-1][7:])
    assert res["tp"] == 2 and res["dp"] == 2 and res["weights"] == "HybridWeights"
    assert res["losses"][2] < res["losses"][0]


ACCUM_WORKER = r'''
import json, os, sys, torch
sys.path.insert(0, %(root)r)
import torch.distributed as dist
from litetorch_b200.models.llama import LlamaConfig
from litetorch_b200.trainer import Trainer
rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
tp = %(tp)d
torch.set_num_threads(2)
cfg = LlamaConfig.tiny()
dp = world // tp
data = torch.randint(0, cfg.vocab_size, (3, dp * 4, 65), generator=torch.Generator().manual_seed(7))
def batch(s):
    d = rank // tp
    return data[s, d * 4:(d + 1) * 4, :-1].contiguous(), data[s, d * 4:(d + 1) * 4, 1:].contiguous()
make = lambda: Trainer(cfg, seed=3, tp=tp, device="cpu", param_dtype=torch.float32, parallel="hybrid" if world > 1 else "none")
a, b = make(), make()
la = [a.step(*batch(s)) for s in range(3)]
lb = [b.step(*batch(s), micro_batches=2) for s in range(3)]
sa = torch.cat([t.flatten().float() for t in a.engine.w.state_tensors().values()])
sb = torch.cat([t.flatten().float() for t in b.engine.w.state_tensors().values()])
if rank == 0:
    print("RESULT " + json.dumps({"la": la, "lb": lb, "diff": float((sa - sb).abs().max())}))
if world > 1:
    dist.barrier()
    dist.destroy_process_group()
'''


@pytest.mark.parametrize("nproc,tp", [(1, 1), (4, 2)])
def test_gradient_accumulation_equals_the_one_batch_step(tmp_path, nproc, tp):
    """`Trainer.step(..., micro_batches=2)`: two half batches accumulated into one AdamW step give the losses and the
    parameters / moments of the whole batch in one pass, on one rank and on dp2 x tp2 gloo ranks."""
    script = os.path.join(str(tmp_path), "accum_worker.py")
    with open(script, "w") as f:
        f.write(ACCUM_WORKER % {"root": ROOT, "tp": tp})
    if nproc == 1:
        cmd = [sys.executable, script]
    else:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(nproc), "--master-addr",
               "127.0.0.1", "--master-port", "29883", script]
    env = dict(os.environ, OMP_NUM_THREADS="2")
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        env.pop(k, None)
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    res = json.loads([l for l in r.stdout.splitlines() if l.startswith("RESULT ")][-1][7:])
    assert all(abs(x - y) < 1e-5 for x, y in zip(res["la"], res["lb"])) and res["diff"] < 1e-4, res


def test_gradient_clipping_scales_the_update_and_skips_non_finite_gradients():
    """`grad_clip` on the unsharded engine: the step equals the one taken with the gradient scaled by hand to the bound,
    the norm before clipping is reported, a bound above the norm changes nothing, and a NaN gradient leaves the
    parameters as they were."""
    import torch
    from litetorch_b200.models.llama import LlamaConfig, LlamaEngine, LocalWeights
    from litetorch_b200.trainer import Trainer
    cfg = LlamaConfig.tiny()
    gen = torch.Generator().manual_seed(5)
    tok = torch.randint(0, cfg.vocab_size, (2, 33), generator=gen)
    x, y = tok[:, :-1], tok[:, 1:]
    mk = lambda clip: LlamaEngine(cfg, "cpu", weights=LocalWeights(cfg, "cpu", seed=3, param_dtype=torch.float32), grad_clip=clip)
    probe = mk(0.0)
    probe.forward_backward(x, y)
    norm = float(probe.w.flat_g.double().norm())
    bound = norm / 4
    clipped, manual, loose = mk(bound), mk(0.0), mk(norm * 10)
    diff = lambda e1, e2: max(float((a - b).abs().max()) for a, b in zip(e1.w.parameters(), e2.w.parameters()))
    probe.optimizer_step()
    for step in range(3):        # Adam's first step does not depend on the gradient's scale: compare over several
        clipped.train_step(x, y)
        if step == 0:
            assert abs(float(clipped.last_grad_norm) - norm) < 1e-5 * norm
        manual.forward_backward(x, y)
        n = float(manual.w.flat_g.double().norm())
        manual.w.flat_g.mul_(min(1.0, bound / (n + 1e-6)))
        manual.optimizer_step()
        loose.train_step(x, y)
        if step:
            probe.train_step(x, y)
    assert diff(clipped, manual) < 1e-6
    assert diff(loose, probe) < 1e-7
    assert diff(clipped, probe) > 1e-5          # the bound did change the trajectory
    # accumulation goes through the same clipping
    acc, one = mk(bound), mk(bound)
    acc.train_step_accumulated([(x[:1], y[:1]), (x[1:], y[1:])])
    one.train_step(x, y)
    assert max(float((a - b).abs().max()) for a, b in zip(acc.w.parameters(), one.w.parameters())) < 1e-5
    # a non-finite gradient: the update is skipped on the device
    bad = mk(bound)
    before = [p.clone() for p in bad.w.parameters()]
    bad.forward_backward(x, y)
    bad.w.flat_g[7] = float("nan")
    bad.optimizer_step(dyn=bad._clip_dyn())
    assert all(torch.equal(a, b) for a, b in zip(before, bad.w.parameters()))
    t = Trainer(cfg, device="cpu", param_dtype=torch.float32, parallel="none", grad_clip=bound, seed=3)
    t.step(x, y)
    assert abs(float(t.engine.last_grad_norm) - norm) < 1e-4 * norm


def test_eval_loss_is_the_training_loss_without_side_effects():
    import torch
    from litetorch_b200.models.llama import LlamaConfig
    from litetorch_b200.trainer import Trainer
    cfg = LlamaConfig.tiny()
    tok = torch.randint(0, cfg.vocab_size, (2, 33), generator=torch.Generator().manual_seed(0))
    x, y = tok[:, :-1], tok[:, 1:]
    t = Trainer(cfg, device="cpu", param_dtype=torch.float32, parallel="none", seed=1)
    t.step(x, y)
    grads, moments, count = t.engine.w.flat_g.clone(), t.engine.w.m.clone(), t.engine.step_count
    before = t.evaluate(x, y)
    assert torch.equal(grads, t.engine.w.flat_g) and torch.equal(moments, t.engine.w.m) and t.engine.step_count == count
    assert abs(before - t.step(x, y)) < 1e-5          # the step reports the loss before its update
    assert t.evaluate(x, y) < before


def test_targets_of_minus_100_are_ignored_in_loss_and_gradient():
    """Masked positions (prompt tokens in supervised fine-tuning) contribute neither loss nor gradient; the mean is over
    all positions, as in the unmasked case."""
    import torch
    from litetorch_b200.models.llama import LlamaConfig, LlamaEngine, LocalWeights, TorchLlama
    cfg = LlamaConfig.tiny()
    e = LlamaEngine(cfg, "cpu", weights=LocalWeights(cfg, "cpu", seed=1, param_dtype=torch.float32))
    tok = torch.randint(0, cfg.vocab_size, (2, 33), generator=torch.Generator().manual_seed(0))
    x, y = tok[:, :-1], tok[:, 1:].clone()
    y[:, :10] = -100
    loss = float(e.forward_backward(x, y))
    ref = TorchLlama(cfg)
    ref.load_from([e.w.p(s.name).float() for s in e.w.specs])
    want = torch.nn.functional.cross_entropy(ref(x).view(-1, cfg.vocab_size), y.reshape(-1), ignore_index=-100, reduction="sum") / y.numel()
    want.backward()
    assert abs(loss - float(want.detach())) < 1e-5 and abs(float(e.eval_loss(x, y)) - loss) < 1e-6
    assert max(float((e.w.g(s.name) - ref.P(s.name).grad).abs().max()) for s in e.w.specs) < 1e-5
