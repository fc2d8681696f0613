"""The small end-to-end demo: a three-armed spiral classified by an MLP through the public `lt.*` API.

    python -m litetorch_b200.models.spiral [--epochs 300] [--device cpu|cuda]

Same workload as the reference's demo (tests/demo_run.py: 600 points on three spiral arms, a 2-64-64-3 MLP, 300 epochs of
full-batch training, then loss, accuracy, memory and time), written against this package: `lt.nn.Sequential`, `lt.optim.AdamW`,
`lt.Ops.cross_entropy_loss`, `Tensor.backward`.  Prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import math
import resource
import time

import torch

import litetorch_b200 as lt
from litetorch_b200.core import _unwrap


def spiral(samples: int = 600, classes: int = 3):
    """Points of `classes` interleaved arms; the radius grows along an arm and a slow ripple keeps the arms from being exact curves."""
    per = samples // classes
    t = torch.linspace(0.0, 1.0, per)
    xs, ys = [], []
    for c in range(classes):
        angle = t * 4.0 * math.pi + c * 2.0 * math.pi / classes
        r = 0.2 + 0.8 * t + 0.03 * torch.sin(11.0 * t + 1.7 * c)
        xs.append(torch.stack([r * torch.cos(angle), r * torch.sin(angle)], 1))
        ys.append(torch.full((per,), float(c)))
    return torch.cat(xs), torch.cat(ys)


def train(epochs: int = 300, device: str = "cpu", hidden: int = 64, lr: float = 1e-2, seed: int = 0):
    lt.manual_seed(seed)
    x, y = spiral()
    dev = lt.Device(device)
    net = lt.nn.Sequential([lt.nn.Linear(2, hidden), lt.nn.Tanh(), lt.nn.Linear(hidden, hidden), lt.nn.Tanh(), lt.nn.Linear(hidden, 3)])
    net.to(dev)
    opt = lt.optim.AdamW(net.parameters(), lr=lr, weight_decay=0.0)
    xs, ys = lt.Tensor.from_torch(x).to(dev), lt.Tensor.from_torch(y).to(dev)
    t0 = time.perf_counter()
    first = last = None
    for _ in range(epochs):
        opt.zero_grad()
        loss = lt.Ops.cross_entropy_loss(net(xs), ys)
        loss.backward()
        opt.step()
        last = loss.item()
        first = last if first is None else first
    seconds = time.perf_counter() - t0
    pred = _unwrap(net(xs)).argmax(-1).cpu()
    acc = float((pred == y.long()).float().mean())
    return {"epochs": epochs, "device": str(dev), "first_loss": round(first, 4), "loss": round(last, 4), "accuracy": round(acc, 4),
            "seconds": round(seconds, 3), "peak_rss_mb": round(resource.getrusage(resource.RUSAGE_SELF).ru_maxrss / 1024.0, 1),
            "gpu_allocated_mb": round(lt.cuda.memory_allocated() / 2 ** 20, 1) if lt.is_gpu_available() else 0.0}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--epochs", type=int, default=300)
    ap.add_argument("--device", default="cuda" if lt.is_gpu_available() else "cpu")
    a = ap.parse_args()
    print(json.dumps(train(a.epochs, a.device)))


if __name__ == "__main__":
    main()
