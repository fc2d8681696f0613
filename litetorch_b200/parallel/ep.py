"""Expert parallelism: a Mixture-of-Experts SwiGLU block whose experts are spread over the EP group.

The reference has a single-process MoE only (src/nn/moe.cpp:11-278) and no all-to-all anywhere.  This block
implements what the MoE configuration asks for: fp32 softmax router, top-k routing with renormalised weights,
capacity factor (tokens beyond an expert's capacity are dropped), the load-balancing auxiliary loss
`E * sum_e f_e * P_e`, data-parallel attention outside, and expert parallelism inside: tokens are dispatched to
the rank that owns their expert, every rank runs its local experts as grouped GEMMs, and the results are
combined back.  Dispatch and combine are autograd-aware all-to-alls (`torch.distributed.all_to_all_single`
over NCCL; the gloo build used for CPU tests emulates it with all-gathers).
"""
from __future__ import annotations

import math
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from ..core import Tensor, _unwrap
from ..ops import functional as Fn


def _world(g) -> int:
    return dist.get_world_size(g) if dist.is_initialized() else 1


def _rank(g) -> int:
    return dist.get_rank(g) if dist.is_initialized() else 0


def _a2a(x: torch.Tensor, out_splits: List[int], in_splits: List[int], group) -> torch.Tensor:
    """Rows of x grouped by destination rank (in_splits) -> rows grouped by source rank (out_splits)."""
    W = _world(group)
    if W == 1:
        return x
    out = x.new_empty((sum(out_splits),) + tuple(x.shape[1:]))
    if x.is_cuda:
        dist.all_to_all_single(out, x.contiguous(), out_splits, in_splits, group=group)
        return out
    # gloo: gather everything, keep what is addressed to this rank
    r = _rank(group)
    sizes = torch.tensor(in_splits, dtype=torch.int64)
    all_sizes = [torch.empty_like(sizes) for _ in range(W)]
    dist.all_gather(all_sizes, sizes, group=group)
    pad = int(max(int(s.sum()) for s in all_sizes))
    buf = x.new_zeros((pad,) + tuple(x.shape[1:]))
    buf[:x.shape[0]] = x
    allbuf = [torch.empty_like(buf) for _ in range(W)]
    dist.all_gather(allbuf, buf, group=group)
    parts = []
    for src in range(W):
        off = int(all_sizes[src][:r].sum())
        parts.append(allbuf[src][off:off + int(all_sizes[src][r])])
    return torch.cat(parts, 0)


class _AllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, out_splits, in_splits, group):
        ctx.out_splits, ctx.in_splits, ctx.group = out_splits, in_splits, group
        return _a2a(x, out_splits, in_splits, group)

    @staticmethod
    def backward(ctx, g):
        return _a2a(g.contiguous(), ctx.in_splits, ctx.out_splits, ctx.group), None, None, None


class MoEFeedForward:
    """SwiGLU experts [E, 2F, d] / [E, d, F]; rank r of the EP group owns experts [r*E/W, (r+1)*E/W)."""

    def __init__(self, dim: int, ffn: int, num_experts: int, top_k: int = 2, capacity_factor: float = 1.25,
                 aux_loss_coef: float = 0.01, group=None, dtype=torch.float32, device="cpu", seed: int = 0, init_std: float = 0.02):
        self.group = group
        W, r = _world(group), _rank(group)
        assert num_experts % W == 0
        self.dim, self.ffn, self.E, self.k = dim, ffn, num_experts, top_k
        self.local_E = num_experts // W
        self.first = r * self.local_E
        self.capacity_factor, self.aux_loss_coef = capacity_factor, aux_loss_coef
        g = torch.Generator().manual_seed(seed)
        self.gate_weight = Tensor(torch.empty(num_experts, dim).normal_(0, init_std, generator=g).to(device).requires_grad_(True))
        w_gu = torch.empty(num_experts, 2 * ffn, dim).normal_(0, init_std, generator=g)
        w_dn = torch.empty(num_experts, dim, ffn).normal_(0, init_std, generator=g)
        sl = slice(self.first, self.first + self.local_E)
        self.w_gate_up = Tensor(w_gu[sl].clone().to(device=device, dtype=dtype).requires_grad_(True))
        self.w_down = Tensor(w_dn[sl].clone().to(device=device, dtype=dtype).requires_grad_(True))
        self.last_aux_loss: Optional[torch.Tensor] = None
        self._dropped = 0
        self.training = True

    def parameters(self):
        return [self.gate_weight, self.w_gate_up, self.w_down]

    @property
    def last_dropped(self) -> int:
        """Slots cut by the capacity limit in the last forward pass."""
        return int(self._dropped)

    def route(self, x2: torch.Tensor):
        """fp32 router. Returns (weights [N,k], experts [N,k], keep mask [N,k], aux loss)."""
        N = x2.shape[0]
        logits = torch.nn.functional.linear(x2.float(), _unwrap(self.gate_weight).float())
        top_w, top_i, probs = Fn.moe_router(logits, self.k, renorm=True)   # warp-per-token kernel on CUDA
        # load balance: f_e = fraction of routed slots on expert e, P_e = mean router probability
        flat = top_i.reshape(-1).long()
        counts = torch.bincount(flat, minlength=self.E)
        f = counts.float() / (N * self.k)
        aux = self.E * (f * probs.mean(0)).sum()
        # capacity: position of each slot inside its expert's queue, in token order.  A stable sort by expert gives the
        # queues directly (a cumulative sum over a one-hot [N k, E] matrix walks the N k rows one after the other on a GPU)
        cap = max(1, int(math.ceil(self.capacity_factor * N * self.k / self.E)))
        order = torch.argsort(flat, stable=True)
        starts = torch.cumsum(counts, 0) - counts
        pos = torch.empty_like(flat)
        pos[order] = torch.arange(flat.numel(), device=flat.device) - starts[flat[order]]
        keep = (pos < cap).view(N, self.k)
        return top_w, top_i, keep, aux

    def forward(self, x: Tensor) -> Tensor:
        xt = _unwrap(x)
        shape = xt.shape
        x2 = xt.reshape(-1, shape[-1])
        N = x2.shape[0]
        W = _world(self.group)
        top_w, top_i, keep, aux = self.route(x2)
        self.last_aux_loss = aux * self.aux_loss_coef
        self._dropped = (~keep).sum()                 # read lazily: no host sync in the step
        # slots that survive the capacity cut, sorted by expert (hence by destination rank)
        slot_tok = torch.arange(N, device=x2.device).repeat_interleave(self.k)[keep.reshape(-1)]
        slot_exp = top_i.reshape(-1)[keep.reshape(-1)]
        slot_w = top_w.reshape(-1)[keep.reshape(-1)]
        order = torch.argsort(slot_exp, stable=True)
        slot_tok, slot_exp, slot_w = slot_tok[order], slot_exp[order], slot_w[order]
        send_counts_e = torch.bincount(slot_exp, minlength=self.E)
        in_splits = send_counts_e.view(W, self.local_E).sum(1).tolist()
        # counts per (source rank, local expert) so that the receiver can regroup by expert
        if W > 1:
            all_counts = [torch.empty_like(send_counts_e) for _ in range(W)]
            dist.all_gather(all_counts, send_counts_e, group=self.group)
            recv_counts = torch.stack([c[self.first:self.first + self.local_E] for c in all_counts], 0)  # [W, local_E]
        else:
            recv_counts = send_counts_e.view(1, self.E)
        out_splits = recv_counts.sum(1).tolist()
        xs = _AllToAll.apply(x2[slot_tok], out_splits, in_splits, self.group)
        # received rows are ordered (source rank, expert); regroup to (expert, source rank)
        rc = recv_counts.tolist()
        src_off = [0]
        for s in range(len(rc)):
            src_off.append(src_off[-1] + sum(rc[s]))
        idx = []
        for e in range(self.local_E):
            for s in range(len(rc)):
                st = src_off[s] + sum(rc[s][:e])
                idx.append(torch.arange(st, st + rc[s][e], device=x2.device))
        perm = torch.cat(idx) if idx else torch.zeros(0, dtype=torch.int64, device=x2.device)
        xe = xs[perm]
        per_e = [sum(rc[s][e] for s in range(len(rc))) for e in range(self.local_E)]
        outs, st = [], 0
        wgu, wdn = _unwrap(self.w_gate_up), _unwrap(self.w_down)
        for e in range(self.local_E):
            c = per_e[e]
            if c:
                h = Fn.swiglu(Fn.linear(xe[st:st + c].to(wgu.dtype), wgu[e]))
                outs.append(Fn.linear(h, wdn[e]))
            st += c
        ye = torch.cat(outs, 0) if outs else xe.new_zeros((0, self.dim))
        inv = torch.empty_like(perm)
        inv[perm] = torch.arange(perm.numel(), device=perm.device)
        ys = _AllToAll.apply(ye[inv].to(x2.dtype), in_splits, out_splits, self.group)
        y = torch.zeros_like(x2).index_add(0, slot_tok, ys * slot_w[:, None].to(ys.dtype))
        return Tensor(y.view(shape))

    __call__ = forward
