"""GPT decoder LM on the public `lt.nn` API: pre-LayerNorm, causal softmax attention with RoPE, GELU MLP.

This is the small CPU/fp32 configuration of the benchmark set (vocab 256, 2 layers, d_model 128, 4 heads,
MLP 512, seq 64, batch 8, AdamW 3e-4 / (0.9, 0.95) / wd 0.1, weights N(0, 0.02), uniform random tokens,
targets = inputs shifted by one):

    python -m litetorch_b200.models.gpt --steps 20

prints the loss curve and tokens/s.  The same module runs on CUDA (bf16 parameters reach the sm_100a
kernels through `lt.Ops`).
"""
from __future__ import annotations

import argparse
import json
import math
import time
from dataclasses import dataclass

import torch

from .. import nn
from ..core import Tensor, _unwrap
from ..ops import Ops
from ..ops import functional as Fn


@dataclass
class GPTConfig:
    vocab_size: int = 256
    n_layers: int = 2
    d_model: int = 128
    n_heads: int = 4
    mlp: int = 512
    max_seq: int = 64
    rope_theta: float = 1e4
    init_std: float = 0.02


class GPTBlock(nn.Module):
    def __init__(self, cfg: GPTConfig):
        super().__init__()
        d = cfg.d_model
        self.n_heads, self.hd = cfg.n_heads, d // cfg.n_heads
        self.ln1, self.ln2 = nn.LayerNorm([d]), nn.LayerNorm([d])
        self.wq, self.wk, self.wv, self.wo = (nn.Linear(d, d, False) for _ in range(4))
        self.fc1, self.fc2 = nn.Linear(d, cfg.mlp, True), nn.Linear(cfg.mlp, d, True)

    def forward(self, x: Tensor, cos: Tensor, sin: Tensor) -> Tensor:
        B, T, d = x.shape
        h = self.ln1(x)
        def heads(t): return _unwrap(t).view(B, T, self.n_heads, self.hd).transpose(1, 2)
        q = Fn.rope(heads(self.wq(h)), _unwrap(cos), _unwrap(sin))
        k = Fn.rope(heads(self.wk(h)), _unwrap(cos), _unwrap(sin))
        v = heads(self.wv(h))
        a = Fn.flash_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(B, T, d)
        x = Ops.add(x, self.wo(Tensor(a)))
        h = self.ln2(x)
        return Ops.add(x, self.fc2(Ops.gelu(self.fc1(h))))


class GPT(nn.Module):
    def __init__(self, cfg: GPTConfig, seed: int = 0):
        super().__init__()
        self.cfg = cfg
        torch.manual_seed(seed)
        self.embed = nn.Embedding(cfg.vocab_size, cfg.d_model)
        self.blocks = [GPTBlock(cfg) for _ in range(cfg.n_layers)]
        self.ln_f = nn.LayerNorm([cfg.d_model])
        self.head = nn.Linear(cfg.d_model, cfg.vocab_size, False)
        hd = cfg.d_model // cfg.n_heads
        inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, hd, 2, dtype=torch.float64) / hd))
        ang = torch.arange(cfg.max_seq, dtype=torch.float64)[:, None] * inv[None]
        self.cos, self.sin = Tensor(ang.cos().float()), Tensor(ang.sin().float())
        with torch.no_grad():
            for p in self.parameters():
                t = _unwrap(p)
                if t.dim() >= 2:
                    t.normal_(0.0, cfg.init_std)
                elif t.numel() and not (t == 1).all():
                    t.zero_()

    def forward(self, tokens: Tensor) -> Tensor:
        x = self.embed(tokens)
        T = x.shape[1]
        cos = Tensor(_unwrap(self.cos)[:T].to(_unwrap(x).device))
        sin = Tensor(_unwrap(self.sin)[:T].to(_unwrap(x).device))
        for b in self.blocks:
            x = b.forward(x, cos, sin)
        return self.head(self.ln_f(x))


def train(steps: int = 20, batch: int = 8, seq: int = 64, device="cpu", seed: int = 0, cfg: GPTConfig = None, verbose=True):
    from .. import optim
    cfg = cfg or GPTConfig()
    model = GPT(cfg, seed).to(device)
    opt = optim.AdamW(model.parameters(), lr=3e-4, beta1=0.9, beta2=0.95, weight_decay=0.1)
    gen = torch.Generator().manual_seed(seed + 1)
    losses, times = [], []
    for step in range(steps):
        seqs = torch.randint(0, cfg.vocab_size, (batch, seq + 1), generator=gen)
        tok = Tensor(seqs[:, :-1].float().to(device))
        tgt = Tensor(seqs[:, 1:].reshape(-1).float().to(device))
        t0 = time.perf_counter()
        opt.zero_grad()
        logits = model(tok)
        loss = Ops.cross_entropy_loss(logits.view([batch * seq, cfg.vocab_size]), tgt)
        loss.backward()
        opt.step()
        losses.append(loss.item())
        times.append(time.perf_counter() - t0)
    med = sorted(times)[len(times) // 2]
    out = {"config": "gpt vocab 256, 2 layers, d 128, 4 heads, mlp 512, seq %d, batch %d, fp32" % (seq, batch), "device": str(device),
           "steps": steps, "losses": [round(l, 4) for l in losses], "median_ms_per_step": round(med * 1e3, 2),
           "tokens_per_s": round(batch * seq / med, 1)}
    if verbose:
        print(json.dumps(out))
    return out


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--device", default="cpu")
    a = ap.parse_args()
    train(a.steps, device=a.device)
