"""Small vision transformer on the public `lt` API, the workload behind the only benchmark table the reference
publishes (ViT on 64 x 64 RGB images, 8 x 8 patches, d 128, 4 heads, batch 32, AdamW 5e-4: train_cat_dog.py:41-52 and
README.md:309-312, seconds per epoch and milliseconds per image on a T4).  The reference's script needs an image
folder that is not in its repository; here the two classes are synthetic (stripes of two orientations plus noise), so
the same measurement runs anywhere:

    python -m litetorch_b200.models.vit [--epochs 3] [--images 2048] [--device cuda]

Model: patch embedding as a strided convolution, learned position embedding, pre-LayerNorm encoder blocks
(non-causal multi-head attention, GELU MLP), mean pooling over the patches, linear head.
"""
from __future__ import annotations

import argparse
import json
import time
from dataclasses import dataclass

import torch

from .. import nn
from ..core import Tensor, _unwrap
from ..ops import Ops


@dataclass
class ViTConfig:
    image_size: int = 64
    channels: int = 3
    patch: int = 8
    d_model: int = 128
    n_heads: int = 4
    n_blocks: int = 2
    mlp: int = 256
    n_classes: int = 2

    @property
    def n_patches(self) -> int:
        return (self.image_size // self.patch) ** 2


class EncoderBlock(nn.Module):
    def __init__(self, cfg: ViTConfig):
        super().__init__()
        self.ln1, self.ln2 = nn.LayerNorm([cfg.d_model]), nn.LayerNorm([cfg.d_model])
        self.attn = nn.MultiHeadAttention(cfg.d_model, cfg.n_heads)
        self.fc1, self.fc2 = nn.Linear(cfg.d_model, cfg.mlp), nn.Linear(cfg.mlp, cfg.d_model)

    def forward(self, x: Tensor) -> Tensor:
        x = Ops.add(x, self.attn(self.ln1(x)))
        return Ops.add(x, self.fc2(Ops.gelu(self.fc1(self.ln2(x)))))


class ViT(nn.Module):
    def __init__(self, cfg: ViTConfig = None, seed: int = 0):
        super().__init__()
        self.cfg = cfg = cfg or ViTConfig()
        torch.manual_seed(seed)
        self.patch_embed = nn.Conv2d(cfg.channels, cfg.d_model, cfg.patch, stride=cfg.patch)
        self.pos = Tensor((torch.randn(1, cfg.n_patches, cfg.d_model) * 0.02).requires_grad_(True))
        self.blocks = [EncoderBlock(cfg) for _ in range(cfg.n_blocks)]
        for i, b in enumerate(self.blocks):
            setattr(self, "block%d" % i, b)                  # registered as sub-modules
        self.ln_f = nn.LayerNorm([cfg.d_model])
        self.head = nn.Linear(cfg.d_model, cfg.n_classes)

    def forward(self, images: Tensor) -> Tensor:
        cfg = self.cfg
        h = _unwrap(self.patch_embed(images))                 # [B, d, H/p, W/p]
        B = h.shape[0]
        x = Tensor(h.reshape(B, cfg.d_model, cfg.n_patches).transpose(1, 2))
        x = Ops.add(x, self.pos)
        for b in self.blocks:
            x = b(x)
        x = self.ln_f(x)
        return self.head(Tensor(_unwrap(x).mean(1)))                # mean over the patches (`Ops.mean` reduces everything)


def synthetic_images(n: int, cfg: ViTConfig, seed: int = 0):
    """Two classes: horizontal or vertical stripes of a random period and phase, plus noise."""
    g = torch.Generator().manual_seed(seed)
    y = torch.randint(0, 2, (n,), generator=g)
    S = cfg.image_size
    t = torch.arange(S).float()
    period = torch.randint(4, 12, (n,), generator=g).float()
    phase = torch.rand(n, generator=g) * 6.28
    wave = torch.sin(t[None, :] * (6.28 / period[:, None]) + phase[:, None])        # [n, S]
    img = torch.where(y[:, None, None].bool(), wave[:, None, :].expand(n, S, S), wave[:, :, None].expand(n, S, S))
    x = img[:, None].expand(n, cfg.channels, S, S) + 0.3 * torch.randn(n, cfg.channels, S, S, generator=g)
    return x.contiguous(), y.float()


def train(epochs: int = 3, images: int = 1024, batch: int = 32, device: str = "cpu", lr: float = 5e-4, cfg: ViTConfig = None,
          seed: int = 0, verbose: bool = True):
    from .. import optim
    cfg = cfg or ViTConfig()
    model = ViT(cfg, seed).to(device)
    opt = optim.AdamW(model.parameters(), lr=lr, weight_decay=0.01)
    x, y = synthetic_images(images, cfg, seed + 1)
    x, y = x.to(device), y.to(device)
    cuda = str(device).startswith("cuda")
    sync = torch.cuda.synchronize if cuda else (lambda: None)
    epoch_s, losses, accs = [], [], []
    for ep in range(epochs):
        perm = torch.randperm(images, generator=torch.Generator().manual_seed(seed + 10 + ep)).to(device)
        sync()
        t0 = time.perf_counter()
        tot, correct, nb = 0.0, 0, 0
        for i in range(0, images - batch + 1, batch):
            idx = perm[i:i + batch]
            xb, yb = Tensor(x[idx]), Tensor(y[idx])
            opt.zero_grad()
            logits = model(xb)
            loss = Ops.cross_entropy_loss(logits, yb)
            loss.backward()
            opt.step()
            tot += loss.item()
            correct += int((_unwrap(logits).argmax(-1).float() == y[idx]).sum())
            nb += 1
        sync()
        epoch_s.append(time.perf_counter() - t0)
        losses.append(tot / nb)
        accs.append(correct / (nb * batch))
    # single-image inference latency
    one = Tensor(x[:1])
    for _ in range(3):
        model(one)
    sync()
    t0 = time.perf_counter()
    for _ in range(20):
        model(one)
    sync()
    infer_ms = (time.perf_counter() - t0) / 20 * 1e3
    out = {"model": "vit %dx%d patch %d d %d heads %d blocks %d" % (cfg.image_size, cfg.image_size, cfg.patch, cfg.d_model,
                                                                  cfg.n_heads, cfg.n_blocks),
           "device": str(device), "images_per_epoch": images // batch * batch, "batch": batch, "data": "synthetic stripes",
           "epoch_s": [round(t, 3) for t in epoch_s], "loss": [round(l, 4) for l in losses], "accuracy": [round(a, 3) for a in accs],
           "inference_ms_per_image": round(infer_ms, 3)}
    if verbose:
        print(json.dumps(out))
    return out


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--epochs", type=int, default=3)
    ap.add_argument("--images", type=int, default=1024)
    ap.add_argument("--device", default="cpu")
    a = ap.parse_args()
    train(a.epochs, a.images, device=a.device)
