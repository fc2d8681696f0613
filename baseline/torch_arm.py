"""Stock-PyTorch stand-in for the headline configuration on one GPU: the same Llama-1.1B (models/llama.TorchLlama:
cuBLAS GEMMs through torch.matmul, library SDPA, eager elementwise ops, torch.optim.AdamW fused) on the same batch,
bf16 parameters.  This is the "NCCL + cuBLAS only" tier the fused kernels are compared against where the reference's
own CUDA path cannot run the configuration.  Prints one JSON line.

    python baseline/torch_arm.py [--steps 5] [--warmup 3] [--tiny]
"""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from litetorch_b200.models.llama import LlamaConfig, TorchLlama   # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--tiny", action="store_true")
    a = ap.parse_args()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    cfg = LlamaConfig.tiny() if a.tiny else LlamaConfig.llama_1b()
    B, T = (2, 256) if a.tiny else (4, 2048)
    torch.manual_seed(0)
    model = TorchLlama(cfg).to(dev)
    with torch.no_grad():                      # initialised on the device: a billion normal samples are slow on the host
        for p in model.parameters():
            (p.fill_(1.0) if p.dim() == 1 else p.normal_(0.0, 0.02))
    model = model.bfloat16()
    opt = torch.optim.AdamW(model.parameters(), lr=3e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, fused=True)
    g = torch.Generator(device=dev).manual_seed(1)

    def step():
        ids = torch.randint(0, cfg.vocab_size, (B, T + 1), device=dev, generator=g)
        logits = model(ids[:, :-1])
        loss = torch.nn.functional.cross_entropy(logits.float().view(-1, cfg.vocab_size), ids[:, 1:].reshape(-1))
        opt.zero_grad(set_to_none=True)
        loss.backward()
        opt.step()
        return loss

    for _ in range(a.warmup):
        loss = step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.steps):
        loss = step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / a.steps
    print(json.dumps({"impl": "stock pytorch (cuBLAS + SDPA + fused AdamW, eager, bf16 parameters)", "model": cfg.name,
                      "global_batch": B, "seq_len": T, "ms_per_step": round(ms, 3), "tokens_per_s": round(B * T / ms * 1e3, 1),
                      "loss": round(float(loss.detach()), 4), "steps": a.steps, "warmup": a.warmup,
                      "max_memory_allocated_gb": round(torch.cuda.max_memory_allocated() / 2 ** 30, 2)}), flush=True)


if __name__ == "__main__":
    main()
