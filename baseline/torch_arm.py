"""Stock-PyTorch stand-in ("NCCL + cuBLAS only" tier) for the benchmark configurations: the same Llama architecture
written as a plain nn.Module - cuBLAS GEMMs through torch.matmul, library scaled_dot_product_attention, eager
elementwise ops, torch.optim.AdamW(fused=True) - sharded with torch's own FSDP2 (`fully_shard`, one group per decoder
layer, bf16 compute with fp32 sharded parameters and fp32 gradient reduction) when run on more than one GPU, and
optionally compiled with torch.compile.  Nothing of this repository's kernels or engine is used; only the model
configuration (sizes) is imported.  It is the number the fused kernels have to beat wherever the reference's own CUDA
path cannot run a configuration.  Prints one JSON line on rank 0.

    python baseline/torch_arm.py --model llama3-8b [--steps 5] [--warmup 3] [--compile] [--ckpt]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 \
        baseline/torch_arm.py --model llama3-8b
"""
import argparse
import json
import os
import sys

import torch
import torch.nn as nn
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from litetorch_b200.models.llama import LlamaConfig   # noqa: E402  (sizes only)

SHAPES = {"llama3-8b": (LlamaConfig.llama3_8b, 1, 8192), "llama-1.1b": (LlamaConfig.llama_1b, 4, 2048),
          "llama-tiny": (LlamaConfig.tiny, 4, 256)}


class RMSNorm(nn.Module):
    def __init__(self, d, eps):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(d))
        self.eps = eps

    def forward(self, x):
        return F.rms_norm(x, (x.shape[-1],), self.weight, self.eps)


def rope(x, cos, sin):
    x0, x1 = x[..., 0::2], x[..., 1::2]
    return torch.stack([x0 * cos - x1 * sin, x0 * sin + x1 * cos], dim=-1).flatten(-2)


class Layer(nn.Module):
    def __init__(self, c):
        super().__init__()
        self.c = c
        self.n1, self.n2 = RMSNorm(c.d_model, c.rms_eps), RMSNorm(c.d_model, c.rms_eps)
        self.wqkv = nn.Linear(c.d_model, c.qkv_dim, bias=False)
        self.wo = nn.Linear(c.n_heads * c.head_dim, c.d_model, bias=False)
        self.w_gu = nn.Linear(c.d_model, 2 * c.ffn, bias=False)
        self.w_down = nn.Linear(c.ffn, c.d_model, bias=False)

    def forward(self, x, cos, sin):
        c = self.c
        B, T, _ = x.shape
        Hq, Hkv, hd = c.n_heads, c.n_kv_heads, c.head_dim
        qkv = self.wqkv(self.n1(x))
        q = qkv[..., :Hq * hd].view(B, T, Hq, hd)
        k = qkv[..., Hq * hd:(Hq + Hkv) * hd].view(B, T, Hkv, hd)
        v = qkv[..., (Hq + Hkv) * hd:].view(B, T, Hkv, hd)
        q, k = rope(q, cos, sin), rope(k, cos, sin)
        o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True, enable_gqa=True)
        x = x + self.wo(o.transpose(1, 2).reshape(B, T, Hq * hd))
        gu = self.w_gu(self.n2(x))
        return x + self.w_down(F.silu(gu[..., :c.ffn]) * gu[..., c.ffn:])


class Llama(nn.Module):
    def __init__(self, c, ckpt=False):
        super().__init__()
        self.c, self.ckpt = c, ckpt
        self.embed = nn.Embedding(c.vocab_size, c.d_model)
        self.layers = nn.ModuleList([Layer(c) for _ in range(c.n_layers)])
        self.norm = RMSNorm(c.d_model, c.rms_eps)
        self.head = nn.Linear(c.d_model, c.vocab_size, bias=False)

    def forward(self, tok):
        c = self.c
        T = tok.shape[1]
        inv = 1.0 / (c.rope_theta ** (torch.arange(0, c.head_dim, 2, device=tok.device, dtype=torch.float32) / c.head_dim))
        ang = torch.arange(T, device=tok.device, dtype=torch.float32)[:, None] * inv[None]
        cos, sin = ang.cos()[None, :, None, :].to(torch.bfloat16), ang.sin()[None, :, None, :].to(torch.bfloat16)
        x = self.embed(tok)
        for l in self.layers:
            if self.ckpt:
                x = torch.utils.checkpoint.checkpoint(l, x, cos, sin, use_reentrant=False)
            else:
                x = l(x, cos, sin)
        return self.head(self.norm(x))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama3-8b", choices=list(SHAPES))
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--compile", action="store_true")
    ap.add_argument("--ckpt", action="store_true", help="recompute every layer in the backward pass")
    a = ap.parse_args()
    world, rank, local = (int(os.environ.get(k, d)) for k, d in (("WORLD_SIZE", 1), ("RANK", 0), ("LOCAL_RANK", 0)))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    make, B, T = SHAPES[a.model]
    cfg = make()
    T = min(T, cfg.max_seq)
    torch.manual_seed(0)
    with torch.device(dev):
        model = Llama(cfg, ckpt=a.ckpt)
    with torch.no_grad():
        for p in model.parameters():
            (p.fill_(1.0) if p.dim() == 1 else p.normal_(0.0, 0.02))
    if world > 1:
        from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard
        mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32)
        for l in model.layers:
            fully_shard(l, mp_policy=mp)
        fully_shard(model, mp_policy=mp)
        layout = "FSDP2 (fully_shard per layer), fp32 sharded parameters, bf16 compute"
    else:
        model = model.bfloat16()
        layout = "single GPU, bf16 parameters (no fp32 master copies)"
    run = torch.compile(model) if a.compile else model
    opt = torch.optim.AdamW(model.parameters(), lr=3e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, fused=True)
    g = torch.Generator(device=dev).manual_seed(1 + rank)

    def step():
        ids = torch.randint(0, cfg.vocab_size, (B, T + 1), device=dev, generator=g)
        logits = run(ids[:, :-1])
        loss = F.cross_entropy(logits.float().view(-1, cfg.vocab_size), ids[:, 1:].reshape(-1))
        opt.zero_grad(set_to_none=True)
        loss.backward()
        opt.step()
        return loss

    for _ in range(a.warmup):
        loss = step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.steps):
        loss = step()
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1) / a.steps], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms = float(ms)
    if rank == 0:
        print(json.dumps({"impl": "stock pytorch (cuBLAS + SDPA + fused AdamW%s)" % (", torch.compile" if a.compile else ", eager"),
                          "layout": layout, "model": cfg.name, "n_gpus": world, "global_batch": B * world, "seq_len": T,
                          "checkpointing": bool(a.ckpt), "ms_per_step": round(ms, 3),
                          "tokens_per_s": round(B * T * world / ms * 1e3, 1), "loss": round(float(loss.detach()), 4),
                          "steps": a.steps, "warmup": a.warmup,
                          "max_memory_allocated_gb": round(torch.cuda.max_memory_allocated() / 2 ** 30, 2)}), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
