"""Mixture-of-experts layers.

`MoELinear(in, out, num_experts, top_k)` is the reference layer (src/nn/moe.cpp:11-278): a softmax gate in
fp32, top-k routing with renormalised weights, and E Linear experts.  Tokens are grouped by expert (sorted
once), every expert runs one GEMM over its own tokens on the tcgen05 path, and the outputs are scattered back
weighted by the gate - instead of the reference's launch of every expert over all tokens with one thread per
token.  The expert-parallel SwiGLU block with capacity factor and load-balancing loss lives in
`litetorch_b200.parallel.ep`.
"""
from __future__ import annotations

import torch

from ..core import Tensor, _unwrap
from ..ops import functional as Fn
from . import Linear, Module  # nn/__init__ imports this file after defining both


def route_top_k(x2: torch.Tensor, gate_w: torch.Tensor, top_k: int):
    """fp32 router: returns (weights [N,k], expert ids [N,k], full probabilities [N,E])."""
    logits = torch.nn.functional.linear(x2.float(), gate_w.float())
    return Fn.moe_router(logits, top_k, renorm=True)


def grouped_expert_apply(x2: torch.Tensor, top_w: torch.Tensor, top_i: torch.Tensor, n_experts: int, expert_fn):
    """y[n] = sum_j w[n,j] * expert_{i[n,j]}(x[n]); tokens are sorted by expert so each expert sees one contiguous
    batch. `expert_fn(e, xs)` maps the [n_e, in] slice of expert e."""
    N, k = top_i.shape
    flat_e = top_i.reshape(-1)
    order = torch.argsort(flat_e, stable=True)
    tok = torch.arange(N, device=x2.device).repeat_interleave(k)[order]
    counts = torch.bincount(flat_e, minlength=n_experts).tolist()
    xs = x2[tok]
    outs, start = [], 0
    for e in range(n_experts):
        c = counts[e]
        if c:
            outs.append(expert_fn(e, xs[start:start + c]))
        start += c
    ys = torch.cat(outs, 0) if outs else xs.new_zeros((0, 0))
    w = top_w.reshape(-1)[order].to(ys.dtype)
    y = torch.zeros((N, ys.shape[1]), dtype=ys.dtype, device=x2.device)
    return y.index_add(0, tok, ys * w[:, None])


class MoELinear(Module):
    def __init__(self, in_features: int, out_features: int, num_experts: int, top_k: int):
        super().__init__()
        self.in_features, self.out_features, self.num_experts, self.top_k = in_features, out_features, num_experts, top_k
        self.gate_weight = Tensor((torch.randn(num_experts, in_features) * 0.02).requires_grad_(True))
        self.experts = [Linear(in_features, out_features, True) for _ in range(num_experts)]

    def forward(self, x: Tensor) -> Tensor:
        xt = _unwrap(x)
        x2 = xt.reshape(-1, xt.shape[-1])
        top_w, top_i, _ = route_top_k(x2, _unwrap(self.gate_weight), self.top_k)

        def run(e, xs):
            lin = self.experts[e]
            return Fn.linear(xs, _unwrap(lin.weight).to(xs.dtype), _unwrap(lin.bias).to(xs.dtype))
        y = grouped_expert_apply(x2, top_w, top_i, self.num_experts, run)
        return Tensor(y.reshape(*xt.shape[:-1], self.out_features))
