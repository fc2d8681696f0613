"""Llama engine (hand-written backward on the sm_100a kernels) against the stock PyTorch model in fp32."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _err(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-9)).item()


@pytest.mark.parametrize("ckpt", [False, True])
def test_engine_matches_torch(ckpt):
    from litetorch_b200.models.llama import LlamaConfig, LlamaEngine, TorchLlama
    from litetorch_b200.ops import kernels as K
    cfg = LlamaConfig.tiny()
    eng = LlamaEngine(cfg, "cuda", seed=3, activation_checkpointing=ckpt)
    ref = TorchLlama(cfg).cuda()
    # oracle uses the bf16-rounded weights the engine computes with, in fp32 arithmetic
    ref.load_from([eng.w.p(s.name).float() for s in eng.w.specs])
    g = torch.Generator(device="cuda").manual_seed(0)
    tok = torch.randint(0, cfg.vocab_size, (2, 200), device="cuda", generator=g)
    tgt = torch.randint(0, cfg.vocab_size, (2, 200), device="cuda", generator=g)
    loss = eng.forward_backward(tok, tgt)
    logits = ref(tok)
    loss_ref = torch.nn.functional.cross_entropy(logits.view(-1, cfg.vocab_size), tgt.view(-1))
    loss_ref.backward()
    torch.cuda.synchronize()
    K.check_status()
    assert abs(loss.item() - loss_ref.item()) < 2e-2
    for s in eng.w.specs:
        e = _err(eng.w.g(s.name), ref.P(s.name).grad)
        assert e < 6e-2, (s.name, e)


def test_loss_decreases_and_matches_adamw():
    from litetorch_b200.models.llama import LlamaConfig, LlamaEngine
    cfg = LlamaConfig.tiny()
    eng = LlamaEngine(cfg, "cuda", seed=1, lr=1e-3)
    g = torch.Generator(device="cuda").manual_seed(0)
    tok = torch.randint(0, cfg.vocab_size, (4, 128), device="cuda", generator=g)
    tgt = torch.roll(tok, -1, 1)
    losses = [float(eng.train_step(tok, tgt)) for _ in range(8)]
    assert losses[-1] < losses[0] - 0.5, losses


def test_trainer_public_api_host_batches():
    from litetorch_b200.models.llama import LlamaConfig
    from litetorch_b200.trainer import Trainer
    cfg = LlamaConfig.tiny()
    tr = Trainer(cfg, device="cuda:0")
    tok = torch.randint(0, cfg.vocab_size, (2, 128)).pin_memory()
    tgt = torch.roll(tok, -1, 1).pin_memory()
    l = tr.step(tok, tgt)
    assert l == l and 4.0 < l < 8.0
    assert tr.h2d_bytes == 2 * 2 * 128 * 8 and tr.d2h_bytes == 4


def test_trainer_from_config_and_metrics_log(tmp_path):
    import json
    from litetorch_b200 import config as C
    from litetorch_b200.trainer import Trainer
    run = C.load("llama-1.1b-fsdp", env={"LT_CFG_MODEL__N_LAYERS": "2", "LT_CFG_MODEL__D_MODEL": "256", "LT_CFG_MODEL__N_Q": "4",
                                         "LT_CFG_MODEL__N_KV": "2", "LT_CFG_MODEL__FFN": "512", "LT_CFG_MODEL__VOCAB": "512",
                                         "LT_CFG_SEQ_LEN": "128"})
    tr = Trainer.from_config(run, device="cuda:0")
    path = str(tmp_path / "metrics.jsonl")
    tr.log_metrics(path)
    tok = torch.randint(0, 512, (2, 128)).pin_memory()
    tgt = torch.roll(tok, -1, 1).pin_memory()
    losses = [tr.step(tok, tgt) for _ in range(3)]
    recs = [json.loads(l) for l in open(path)]
    assert [r["step"] for r in recs] == [1, 2, 3] and abs(recs[2]["loss"] - losses[2]) < 1e-6
    assert recs[1]["tokens_per_s"] > 0 and recs[1]["max_memory_allocated_mb"] > 0
    assert losses[2] < losses[0]


def test_trainer_save_then_load_continues_the_loss_curve(tmp_path):
    """The benchmarked path (Trainer -> LlamaEngine -> flat bf16 weights, fp32 master + AdamW moments, step count)
    saved after step 3 and loaded into a trainer with other weights: the resumed losses equal the uninterrupted run."""
    from litetorch_b200.models.llama import LlamaConfig
    from litetorch_b200.trainer import Trainer
    cfg = LlamaConfig.tiny()
    g = torch.Generator().manual_seed(3)
    data = torch.randint(0, cfg.vocab_size, (6, 2, 129), generator=g)
    batch = lambda s: (data[s, :, :-1].contiguous(), data[s, :, 1:].contiguous())  # noqa: E731
    a = Trainer(cfg, seed=5, parallel="none")
    full = [a.step(*batch(s)) for s in range(6)]
    b = Trainer(cfg, seed=5, parallel="none")
    first = [b.step(*batch(s)) for s in range(3)]
    b.save(str(tmp_path / "ck"))
    c = Trainer(cfg, seed=9, parallel="none")
    c.step(*batch(5))
    c.load(str(tmp_path / "ck"))
    rest = [c.step(*batch(s)) for s in range(3, 6)]
    assert all(abs(x - y) < 2e-3 for x, y in zip(first, full[:3])), (first, full[:3])   # atomics: not bit-reproducible
    assert all(abs(x - y) < 2e-3 for x, y in zip(rest, full[3:])), (rest, full[3:])   # bf16 atomics in two kernels
    assert c.engine.step_count == 6


def test_chunked_head_and_fused_linear_cross_entropy_never_hold_full_logits():
    """The chunked LM head of the engine and `Ops.fused_linear_cross_entropy` on the kernels: same loss and gradients as
    the unchunked path / an fp32 PyTorch reference, with a peak allocation far below the [N, V] logits."""
    import litetorch_b200 as lt
    from litetorch_b200.core import Tensor, _unwrap
    from litetorch_b200.models.llama import LlamaConfig, LlamaEngine
    cfg = LlamaConfig.tiny()
    g = torch.Generator(device="cuda").manual_seed(1)
    tok = torch.randint(0, cfg.vocab_size, (2, 256), device="cuda", generator=g)
    tgt = torch.roll(tok, -1, 1)
    a = LlamaEngine(cfg, "cuda", seed=2)
    b = LlamaEngine(cfg, "cuda", seed=2, head_chunk_rows=128)
    la, lb = a.forward_backward(tok, tgt), b.forward_backward(tok, tgt)
    assert abs(float(la) - float(lb)) < 2e-3
    assert _err(b.w.flat_g, a.w.flat_g) < 2e-2
    # the op: N x V = 8192 x 32768 logits would be 512 MB in bf16; chunks of 1024 rows keep 64 MB at a time
    N, Kd, V = 8192, 256, 32768
    x = (torch.randn(N, Kd, device="cuda", generator=g) * 0.5).bfloat16().requires_grad_(True)
    w = (torch.randn(V, Kd, device="cuda", generator=g) * 0.05).bfloat16().requires_grad_(True)
    t = torch.randint(0, V, (N,), device="cuda", generator=g)
    torch.cuda.synchronize()
    torch.cuda.reset_peak_memory_stats()
    base = torch.cuda.memory_allocated()
    loss = _unwrap(lt.Ops.fused_linear_cross_entropy(Tensor(x), Tensor(w), Tensor(t.float()), chunk_rows=1024))
    loss.sum().backward()
    torch.cuda.synchronize()
    peak = torch.cuda.max_memory_allocated() - base
    assert peak < 0.5 * N * V * 2, peak
    xf, wf = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    ref = torch.nn.functional.cross_entropy(xf @ wf.t(), t)
    ref.backward()
    assert abs(float(loss) - float(ref)) < 2e-3
    assert _err(x.grad, xf.grad) < 2e-2 and _err(w.grad, wf.grad) < 2e-2
