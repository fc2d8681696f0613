"""Stress cases in the spirit of the reference's stress bundle (tests/stress_test.cpp:36-214, tests/memory_leak_test.cpp):
eight threads training at once, resident memory over many iterations, shape-mismatch errors and NaN / Inf propagation."""
import resource
import threading

import pytest
import torch

import litetorch_b200 as lt
from litetorch_b200.core import _unwrap


def _spiral(n, seed):
    g = torch.Generator().manual_seed(seed)
    r = torch.rand(n, generator=g)
    cls = torch.randint(0, 2, (n,), generator=g)
    ang = r * 6.0 + cls * 3.14159
    x = torch.stack([r * torch.cos(ang), r * torch.sin(ang)], 1) + 0.02 * torch.randn(n, 2, generator=g)
    return x, cls.float()


def _train(seed, steps, out, idx):
    x, y = _spiral(256, seed)
    net = lt.nn.Sequential([lt.nn.Linear(2, 32), lt.nn.GELU(), lt.nn.Linear(32, 32), lt.nn.GELU(), lt.nn.Linear(32, 2)])
    opt = lt.optim.AdamW(net.parameters(), lr=1e-2, weight_decay=0.0)
    xs, ys = lt.Tensor.from_torch(x), lt.Tensor.from_torch(y)
    losses = []
    for _ in range(steps):
        opt.zero_grad()
        loss = lt.Ops.cross_entropy_loss(net(xs), ys)
        loss.backward()
        opt.step()
        losses.append(loss.item())
    out[idx] = losses


def test_eight_threads_train_concurrently():
    out = [None] * 8
    ts = [threading.Thread(target=_train, args=(i, 150, out, i)) for i in range(8)]
    for t in ts:
        t.start()
    for t in ts:
        t.join()
    for losses in out:
        assert losses is not None and all(l == l for l in losses)
        assert min(losses[-10:]) < 0.9 * losses[0], (losses[0], losses[-1])


def test_resident_memory_is_flat_over_many_iterations():
    x, y = _spiral(128, 0)
    net = lt.nn.Sequential([lt.nn.Linear(2, 64), lt.nn.GELU(), lt.nn.Linear(64, 2)])
    opt = lt.optim.AdamW(net.parameters(), lr=1e-3)
    xs, ys = lt.Tensor.from_torch(x), lt.Tensor.from_torch(y)

    def run(n):
        for _ in range(n):
            opt.zero_grad()
            loss = lt.Ops.cross_entropy_loss(net(xs), ys)
            loss.backward()
            opt.step()
    run(200)                                                     # warm-up: pools and caches reach their steady size
    before = resource.getrusage(resource.RUSAGE_SELF).ru_maxrss  # KiB on Linux
    run(1000)
    after = resource.getrusage(resource.RUSAGE_SELF).ru_maxrss
    assert after - before < 32 * 1024, (before, after)           # the peak may not grow by more than 32 MiB


def test_shape_mismatch_raises_and_nan_inf_propagate():
    a = lt.Tensor.from_torch(torch.randn(3, 4))
    b = lt.Tensor.from_torch(torch.randn(5, 6))
    with pytest.raises(Exception):
        lt.Ops.matmul(a, b)
    with pytest.raises(Exception):
        lt.Ops.add(a, b)
    with pytest.raises(Exception):
        lt.nn.Linear(7, 3)(a)
    bad = lt.Tensor.from_torch(torch.tensor([1.0, float("nan"), float("inf"), -float("inf")]))
    r = _unwrap(lt.Ops.relu(bad))
    assert r[1] != r[1] and r[2] == float("inf") and r[3] == 0
    s = lt.Ops.sum(lt.Ops.mul(bad, bad))
    assert s.item() != s.item()
    # a non-finite gradient is caught by the scaler and the step is skipped
    w = lt.Tensor.from_torch(torch.ones(2), requires_grad=True) if "requires_grad" in lt.Tensor.from_torch.__code__.co_varnames \
        else lt.Tensor(torch.ones(2, requires_grad=True))
    opt = lt.optim.SGD([w], lr=0.1)
    scaler = lt.amp.GradScaler(init_scale=4.0)
    _unwrap(w).grad = torch.tensor([float("inf"), 1.0])
    scaler.step(opt)
    scaler.update()
    assert torch.equal(_unwrap(w).detach(), torch.ones(2)) and scaler.get_scale() < 4.0


def test_spiral_demo_learns_the_three_arms():
    """The end-to-end demo of the reference's tests/demo_run.py through this package's public API."""
    from litetorch_b200.models.spiral import train
    r = train(epochs=300, device="cpu")
    assert r["loss"] < 0.2 * r["first_loss"] and r["accuracy"] > 0.95, r
