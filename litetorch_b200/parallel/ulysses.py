"""Ulysses sequence parallelism: attention over a sequence-sharded activation by switching to head sharding.

The reference has no all-to-all collective and no Ulysses path (its only sequence-scaling mechanisms are the CPU ring
attention of src/ops/ring_attention.cpp:49-126 and the unused slicing helpers of src/distributed/context_parallel.cpp),
so this is an addition next to the ring attention of `parallel/cp.py`: where ring attention moves KV tiles and keeps
every head on every rank, Ulysses moves activations twice per attention and keeps every rank's kernel a plain,
full-sequence FlashAttention over H / W heads - the better trade when heads are plentiful and the sequence is short
enough that one GPU can hold T x (H / W) x D.

Layout: q [B, T/W, Hq, D], k / v [B, T/W, Hkv, D] with the sequence split contiguously over the group (rank r holds
positions [r T/W, (r+1) T/W)); Hq and Hkv must be multiples of the group size.  All-to-all #1 turns them into
[B, T, H/W, D]; attention runs locally (causal masks need no adjustment, every rank sees whole sequences); all-to-all #2
brings the output back to [B, T/W, Hq, D].  Both exchanges are differentiable (their backward is the opposite exchange).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from ..ops import functional as Fn
from .ep import _a2a, _rank, _world


class _SeqToHead(torch.autograd.Function):
    """[B, T/W, H, D] sharded by sequence -> [B, T, H/W, D] sharded by heads."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _seq_to_head(x, group)

    @staticmethod
    def backward(ctx, g):
        return _head_to_seq(g.contiguous(), ctx.group), None


class _HeadToSeq(torch.autograd.Function):
    """[B, T, H/W, D] sharded by heads -> [B, T/W, H, D] sharded by sequence."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _head_to_seq(x, group)

    @staticmethod
    def backward(ctx, g):
        return _seq_to_head(g.contiguous(), ctx.group), None


def _seq_to_head(x: torch.Tensor, group) -> torch.Tensor:
    W = _world(group)
    if W == 1:
        return x
    B, Tl, H, D = x.shape
    assert H % W == 0, "heads must divide over the Ulysses group"
    Hl = H // W
    # rows grouped by destination rank: destination w gets heads [w Hl, (w+1) Hl) of the local positions
    send = x.reshape(B, Tl, W, Hl, D).permute(2, 0, 1, 3, 4).contiguous().view(W * B, Tl, Hl, D)
    recv = _a2a(send, [B] * W, [B] * W, group)             # [source rank, B, Tl, Hl, D]
    return recv.view(W, B, Tl, Hl, D).permute(1, 0, 2, 3, 4).reshape(B, W * Tl, Hl, D)


def _head_to_seq(x: torch.Tensor, group) -> torch.Tensor:
    W = _world(group)
    if W == 1:
        return x
    B, T, Hl, D = x.shape
    assert T % W == 0
    Tl = T // W
    send = x.reshape(B, W, Tl, Hl, D).permute(1, 0, 2, 3, 4).contiguous().view(W * B, Tl, Hl, D)
    recv = _a2a(send, [B] * W, [B] * W, group)             # [source rank = head group, B, Tl, Hl, D]
    return recv.view(W, B, Tl, Hl, D).permute(1, 2, 0, 3, 4).reshape(B, Tl, W * Hl, D)


def seq_to_head(x: torch.Tensor, group=None) -> torch.Tensor:
    return _SeqToHead.apply(x, group)


def head_to_seq(x: torch.Tensor, group=None) -> torch.Tensor:
    return _HeadToSeq.apply(x, group)


def ulysses_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, group=None, causal: bool = True,
                      scale: Optional[float] = None) -> torch.Tensor:
    """Attention over sequence shards.  q [B, T/W, Hq, D], k / v [B, T/W, Hkv, D] -> [B, T/W, Hq, D]."""
    if not dist.is_initialized() or _world(group) == 1:
        return Fn.flash_attention_bthd(q, k, v, causal, scale)
    W = _world(group)
    if k.shape[2] % W != 0:
        # fewer KV heads than ranks: repeat them so that every rank owns the KV head of its query heads
        rep = W // k.shape[2] if W % k.shape[2] == 0 else None
        assert rep is not None and q.shape[2] % W == 0, "KV heads and group size must divide one another"
        k, v = k.repeat_interleave(rep, 2), v.repeat_interleave(rep, 2)
    o = Fn.flash_attention_bthd(seq_to_head(q, group), seq_to_head(k, group), seq_to_head(v, group), causal, scale)
    return head_to_seq(o, group)


__all__ = ["ulysses_attention", "seq_to_head", "head_to_seq"]
