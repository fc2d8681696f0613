"""Gradient clipping of the unsharded Llama engine on the device: the norm kernel against a float64 norm, the clipped
trajectory against one whose multiplier is computed on the host, and the skipped update on a non-finite gradient."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_clipped_steps_follow_the_host_computed_multiplier():
    from litetorch_b200.models.llama import LlamaConfig, LlamaEngine
    from litetorch_b200.ops import kernels as K
    cfg = LlamaConfig.tiny()
    g = torch.Generator(device="cuda").manual_seed(0)
    tok = torch.randint(0, cfg.vocab_size, (2, 200), device="cuda", generator=g)
    tgt = torch.randint(0, cfg.vocab_size, (2, 200), device="cuda", generator=g)
    probe = LlamaEngine(cfg, "cuda", seed=3)
    probe.forward_backward(tok, tgt)
    norm = float(probe.w.flat_g.double().norm())
    bound = norm / 4
    clipped, manual = LlamaEngine(cfg, "cuda", seed=3, grad_clip=bound), LlamaEngine(cfg, "cuda", seed=3)
    start = [p.clone() for p in clipped.w.parameters()]
    for step in range(3):
        clipped.train_step(tok, tgt)
        if step == 0:
            assert abs(float(clipped.last_grad_norm) - norm) < 1e-3 * norm
        manual.forward_backward(tok, tgt)
        n = float(manual.w.flat_g.double().norm())
        dyn = torch.tensor([min(1.0, bound / (n + 1e-6)), 0.0, n], dtype=torch.float32, device="cuda")
        manual.optimizer_step(dyn=dyn)
    torch.cuda.synchronize()
    K.check_status()
    moved = sum(float((a - b).double().pow(2).sum()) for a, b in zip(clipped.w.parameters(), start)) ** 0.5
    apart = sum(float((a - b).double().pow(2).sum()) for a, b in zip(clipped.w.parameters(), manual.w.parameters())) ** 0.5
    assert moved > 0 and apart < 0.05 * moved, (moved, apart)


def test_a_non_finite_gradient_skips_the_update():
    from litetorch_b200.models.llama import LlamaConfig, LlamaEngine
    cfg = LlamaConfig.tiny()
    g = torch.Generator(device="cuda").manual_seed(1)
    tok = torch.randint(0, cfg.vocab_size, (2, 128), device="cuda", generator=g)
    tgt = torch.randint(0, cfg.vocab_size, (2, 128), device="cuda", generator=g)
    eng = LlamaEngine(cfg, "cuda", seed=3, grad_clip=1.0)
    before = [p.clone() for p in eng.w.parameters()]
    eng.forward_backward(tok, tgt)
    eng.w.flat_g[7] = float("nan")
    eng.optimizer_step(dyn=eng._clip_dyn())
    torch.cuda.synchronize()
    assert all(torch.equal(a, b) for a, b in zip(before, eng.w.parameters()))
