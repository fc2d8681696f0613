"""Tensor parallelism with optional sequence parallelism: `ColumnParallelLinear`, `RowParallelLinear`.

Reference (src/nn/parallel_linear.cpp:9-116): Column splits W by output rows and all-gathers the outputs, Row
splits W by input columns and all-reduces; both collectives sit OUTSIDE autograd there (the graph is cut).
Here every collective is an autograd function with the matching backward collective, and with
`sequence_parallel=True` the activations between the two layers stay sharded along the sequence:
Column all-gathers its input (backward: reduce-scatter), Row reduce-scatters its output (backward:
all-gather).  On CUDA bf16 with a symmetric-memory context the Column all-gather is fused into the GEMM
(`lt_ag_gemm_bf16`, operand A gathered by M blocks) and the Row reduce-scatter is fused into the GEMM
epilogue (`lt_gemm_rs_bf16`).
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.distributed as dist

from ..core import Tensor, _unwrap
from ..ops import functional as Fn


def _world(group=None) -> int:
    return dist.get_world_size(group) if dist.is_initialized() else 1


def _rank(group=None) -> int:
    return dist.get_rank(group) if dist.is_initialized() else 0


def _all_gather_cat(x: torch.Tensor, dim: int, group) -> torch.Tensor:
    W = _world(group)
    if W == 1:
        return x
    parts = [torch.empty_like(x) for _ in range(W)]
    dist.all_gather(parts, x.contiguous(), group=group)
    return torch.cat(parts, dim)


def _reduce_scatter_dim(x: torch.Tensor, dim: int, group) -> torch.Tensor:
    W = _world(group)
    if W == 1:
        return x
    x = x.contiguous()
    if x.is_cuda:
        chunks = [c.contiguous() for c in x.chunk(W, dim)]
        out = torch.empty_like(chunks[0])
        dist.reduce_scatter(out, chunks, group=group)
        return out
    y = x.clone()
    dist.all_reduce(y, group=group)
    return y.chunk(W, dim)[_rank(group)].contiguous()


class _GatherFwdScatterBwd(torch.autograd.Function):
    """all-gather along `dim`; backward: reduce-scatter (sequence parallel entry) or slice (plain output gather)."""

    @staticmethod
    def forward(ctx, x, dim, group, reduce_in_bwd):
        ctx.dim, ctx.group, ctx.reduce = dim, group, reduce_in_bwd
        return _all_gather_cat(x, dim, group)

    @staticmethod
    def backward(ctx, g):
        if ctx.reduce:
            return _reduce_scatter_dim(g, ctx.dim, ctx.group), None, None, None
        return g.chunk(_world(ctx.group), ctx.dim)[_rank(ctx.group)].contiguous(), None, None, None


class _ScatterFwdGatherBwd(torch.autograd.Function):
    """reduce-scatter along `dim`; backward: all-gather."""

    @staticmethod
    def forward(ctx, x, dim, group):
        ctx.dim, ctx.group = dim, group
        return _reduce_scatter_dim(x, dim, group)

    @staticmethod
    def backward(ctx, g):
        return _all_gather_cat(g, ctx.dim, ctx.group), None, None


class _AllReduceFwd(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        if _world(group) > 1:
            x = x.clone()
            dist.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        return g, None


class _CopyFwdAllReduceBwd(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, g):
        if _world(ctx.group) > 1:
            g = g.clone()
            dist.all_reduce(g, group=ctx.group)
        return g, None


def _init_full(out_f, in_f, seed_shift=0):
    g = torch.Generator().manual_seed(1234 + seed_shift)
    bound = 1.0 / math.sqrt(in_f) if in_f > 0 else 0.0
    return torch.empty(out_f, in_f).uniform_(-bound, bound, generator=g)


class ColumnParallelLinear:
    """y = x W^T + b with W [out, in] split by output rows over the TP group.

    gather_output=True (reference behaviour) returns the full [.., out]; False leaves [.., out/W] for a following
    RowParallelLinear.  sequence_parallel=True expects x sharded on dim 0 ... in [T/W, .., in] layout, i.e. the
    sequence dimension first."""

    def __init__(self, in_features: int, out_features: int, has_bias: bool = True, gather_output: bool = True,
                 sequence_parallel: bool = False, group=None):
        self.group = group
        W, r = _world(group), _rank(group)
        assert out_features % W == 0
        self.in_features, self.out_features, self.local_out = in_features, out_features, out_features // W
        full = _init_full(out_features, in_features)
        self.weight = Tensor(full[r * self.local_out:(r + 1) * self.local_out].clone().requires_grad_(True))
        bound = 1.0 / math.sqrt(in_features)
        fb = torch.empty(out_features).uniform_(-bound, bound, generator=torch.Generator().manual_seed(4321))
        self.bias = Tensor(fb[r * self.local_out:(r + 1) * self.local_out].clone().requires_grad_(True)) if has_bias else None
        self.gather_output, self.sequence_parallel = gather_output, sequence_parallel
        self.training = True
        self.fused = None  # set by parallel.tp_fused.attach() on CUDA

    def forward(self, x: Tensor) -> Tensor:
        xt = _unwrap(x)
        w = _unwrap(self.weight).to(xt.dtype)
        b = _unwrap(self.bias).to(xt.dtype) if self.bias is not None else None
        if self.sequence_parallel:
            if self.fused is not None and xt.is_cuda and xt.dtype == torch.bfloat16:
                y = self.fused.ag_linear(xt, w, b)
            else:
                y = Fn.linear(_GatherFwdScatterBwd.apply(xt, 0, self.group, True), w, b)
        else:
            y = Fn.linear(_CopyFwdAllReduceBwd.apply(xt, self.group), w, b)
        if self.gather_output:
            y = _GatherFwdScatterBwd.apply(y, y.dim() - 1, self.group, False)
        return Tensor(y)

    __call__ = forward

    def parameters(self):
        return [self.weight] + ([self.bias] if self.bias is not None else [])

    def children(self):
        return []

    def to(self, device):
        from ..core import _as_device
        d = _as_device(device)
        self.weight = Tensor(_unwrap(self.weight).detach().to(d).requires_grad_(True))
        if self.bias is not None:
            self.bias = Tensor(_unwrap(self.bias).detach().to(d).requires_grad_(True))
        return self

    def train(self, mode=True):
        self.training = mode
        return self

    def eval(self):
        return self.train(False)


class RowParallelLinear:
    """y = x W^T + b with W [out, in] split by input columns; each rank multiplies its slice of the features and the
    partial results are summed (all-reduce) or, under sequence parallelism, reduce-scattered along the sequence.

    input_is_parallel=False (reference behaviour) takes the full x and slices it locally."""

    def __init__(self, in_features: int, out_features: int, has_bias: bool = True, input_is_parallel: bool = False,
                 sequence_parallel: bool = False, group=None):
        self.group = group
        W, r = _world(group), _rank(group)
        assert in_features % W == 0
        self.in_features, self.out_features, self.local_in = in_features, out_features, in_features // W
        full = _init_full(out_features, in_features, 1)
        self.weight = Tensor(full[:, r * self.local_in:(r + 1) * self.local_in].clone().requires_grad_(True))
        self.bias = Tensor(torch.zeros(out_features).requires_grad_(True)) if has_bias else None
        self.input_is_parallel, self.sequence_parallel = input_is_parallel, sequence_parallel
        self.training = True
        self.fused = None

    def forward(self, x: Tensor) -> Tensor:
        xt = _unwrap(x)
        W, r = _world(self.group), _rank(self.group)
        if not self.input_is_parallel and W > 1:
            xt = xt[..., r * self.local_in:(r + 1) * self.local_in]
        w = _unwrap(self.weight).to(xt.dtype)
        if self.sequence_parallel:
            if self.fused is not None and xt.is_cuda and xt.dtype == torch.bfloat16:
                y = self.fused.linear_rs(xt, w)
            else:
                y = _ScatterFwdGatherBwd.apply(Fn.linear(xt, w), 0, self.group)
        else:
            y = _AllReduceFwd.apply(Fn.linear(xt, w), self.group)
        if self.bias is not None:
            y = y + _unwrap(self.bias).to(y.dtype)
        return Tensor(y)

    __call__ = forward
    parameters = ColumnParallelLinear.parameters
    children = ColumnParallelLinear.children
    to = ColumnParallelLinear.to
    train = ColumnParallelLinear.train
    eval = ColumnParallelLinear.eval


def vocab_parallel_cross_entropy(logits_local: torch.Tensor, targets: torch.Tensor, vocab_start: int, group=None,
                                 ignore_index: int = -100) -> torch.Tensor:
    """Mean CE when the vocabulary is split over the TP group: each rank computes (max, sum-exp, target logit) of its
    shard, ONE small all-gather combines them, and the gradient is written in place on each rank's shard."""
    return _VocabParallelCE.apply(logits_local, targets, vocab_start, group, ignore_index)


class _VocabParallelCE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, targets, vocab_start, group, ignore_index):
        N, V = logits.shape
        tgt = targets.to(torch.int64)
        n_valid = max(int((tgt != ignore_index).sum().item()), 1)
        native = logits.is_cuda and logits.dtype == torch.bfloat16
        if native:
            from ..ops import kernels as K
            work = logits.contiguous().clone()
            stats = K.ce_stats(work, tgt, vocab_start)
        else:
            lf = logits.float()
            m = lf.amax(-1)
            s = torch.exp(lf - m[:, None]).sum(-1)
            loc = tgt - vocab_start
            inside = (loc >= 0) & (loc < V)
            tl = torch.where(inside, lf.gather(1, loc.clamp(0, V - 1)[:, None])[:, 0], torch.zeros_like(m))
            stats = torch.stack([m, s, tl], 1)
        W = _world(group)
        if W > 1:
            allst = [torch.empty_like(stats) for _ in range(W)]
            dist.all_gather(allst, stats.contiguous(), group=group)
            st = torch.stack(allst, 0)
            gm = st[:, :, 0].amax(0)
            gs = (st[:, :, 1] * torch.exp(st[:, :, 0] - gm[None])).sum(0)
            gt = st[:, :, 2].sum(0)
            gstats = torch.stack([gm, gs, gt], 1).contiguous()
        else:
            gstats = stats
        if native:
            rows = K.ce_finish(work, tgt, gstats, vocab_start=vocab_start, grad_scale=1.0 / n_valid, ignore_index=ignore_index)
            ctx.save_for_backward(work)
            loss = rows.sum() / n_valid
        else:
            valid = tgt != ignore_index
            rows = torch.where(valid, torch.log(gstats[:, 1]) + gstats[:, 0] - gstats[:, 2], torch.zeros_like(gstats[:, 0]))
            p = torch.exp(logits.float() - gstats[:, 0:1]) / gstats[:, 1:2]
            loc = tgt - vocab_start
            inside = (loc >= 0) & (loc < V) & valid
            p[torch.arange(N, device=p.device)[inside], loc[inside]] -= 1.0
            p = p * valid[:, None] / n_valid
            ctx.save_for_backward(p.to(logits.dtype))
            loss = rows.sum() / n_valid
        return loss

    @staticmethod
    def backward(ctx, g):
        (d,) = ctx.saved_tensors
        return d * g.to(d.dtype), None, None, None, None
