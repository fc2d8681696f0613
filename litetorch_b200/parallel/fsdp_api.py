"""Generic FSDP wrappers of the reference API for arbitrary `lt.nn.Module`s.

* `FullyShardedDataParallel(module)` with `gather_parameters()`, `shard_parameters()`, `get_module()`:
  every parameter is flattened, padded to a multiple of the world size and split into equal shards
  (include/litetorch/fsdp.h:22-130).
* `FSDP.fully_shard(module)`: hook-based ZeRO-3 - leaf modules all-gather their parameters in a forward
  pre-hook, free them after forward, re-gather for backward and reduce-scatter the gradients into the shard in a
  gradient hook (src/distributed/fsdp_wrapper.cpp:12-156; documented in the reference README but not bound to
  Python there).
The Llama engine does not go through these hooks: it uses `ShardedWeights` (fsdp.py), where the gathers and the
reduce-scatter are fused into the GEMM and optimizer kernels.
"""
from __future__ import annotations

from typing import List

import torch
import torch.distributed as dist

from ..core import Tensor, _unwrap


def _world():
    return dist.get_world_size() if dist.is_initialized() else 1


def _rank():
    return dist.get_rank() if dist.is_initialized() else 0


def _shard_of(t: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    n = t.numel()
    per = (n + world - 1) // world
    flat = torch.zeros(per * world, dtype=t.dtype, device=t.device)
    flat[:n] = t.detach().reshape(-1)
    return flat[rank * per:(rank + 1) * per].clone()


def _gather_full(shard: torch.Tensor, shape, world: int) -> torch.Tensor:
    if world == 1:
        full = shard
    else:
        parts = [torch.empty_like(shard) for _ in range(world)]
        dist.all_gather(parts, shard.contiguous())
        full = torch.cat(parts)
    n = 1
    for s in shape:
        n *= s
    return full[:n].view(*shape)


class FullyShardedDataParallel:
    def __init__(self, module):
        self.module = module
        self.world, self.rank = _world(), _rank()
        self.params: List[Tensor] = list(module.parameters())
        self.shapes = [list(_unwrap(p).shape) for p in self.params]
        for p in self.params:
            p.shard = Tensor(_shard_of(_unwrap(p), self.rank, self.world).requires_grad_(True))
        self.sharded = False
        self.shard_parameters()

    def get_module(self):
        return self.module

    def gather_parameters(self) -> None:
        """All-gather every shard into a fresh full parameter (the layout `forward` expects)."""
        for p, shape in zip(self.params, self.shapes):
            full = _gather_full(_unwrap(p.shard).detach(), shape, self.world)
            with torch.no_grad():
                _unwrap(p).data = full.clone()
        self.sharded = False

    def shard_parameters(self) -> None:
        """Keep only this rank's shard: gradients of the full parameter are reduce-scattered into `shard.grad`
        and the full storage is released (the parameter aliases its flat shard)."""
        for p in self.params:
            t = _unwrap(p)
            if t.grad is not None:
                g = t.grad.reshape(-1)
                per = _unwrap(p.shard).numel()
                padded = torch.zeros(per * self.world, dtype=g.dtype, device=g.device)
                padded[:g.numel()] = g
                if self.world > 1:
                    dist.all_reduce(padded)
                _unwrap(p.shard).grad = padded[self.rank * per:(self.rank + 1) * per].clone()
                t.grad = None
            if not self.sharded:
                with torch.no_grad():
                    _unwrap(p.shard).data.copy_(_shard_of(t, self.rank, self.world))
            # the parameter itself now views this rank's flat shard (reference: fsdp.h:113-120), so its shape is
            # [shard_size] until the next gather
            t.data = _unwrap(p.shard).data
        self.sharded = True

    def forward(self, x):
        self.gather_parameters()
        return self.module(x)

    __call__ = forward

    def parameters(self):
        return self.params


class FSDP:
    @staticmethod
    def fully_shard(module):
        """Install the gather / free / reduce-scatter hooks on every leaf module; returns the module."""
        world, rank = _world(), _rank()

        def leaves(m):
            ch = m.children() if hasattr(m, "children") else []
            if not ch:
                yield m
            for c in ch:
                yield from leaves(c)

        for leaf in leaves(module):
            own = [(k, v) for k, v in vars(leaf).items() if isinstance(v, Tensor) and _unwrap(v).requires_grad]
            if not own:
                continue
            state = []
            for k, p in own:
                t = _unwrap(p)
                shape = list(t.shape)
                p.shard = Tensor(_shard_of(t, rank, world))
                state.append((p, shape))

                def make_hook(p=p, shape=shape):
                    def hook(g):
                        flat = g.reshape(-1)
                        per = _unwrap(p.shard).numel()
                        padded = torch.zeros(per * world, dtype=flat.dtype, device=flat.device)
                        padded[:flat.numel()] = flat
                        if world > 1:
                            dist.all_reduce(padded)
                        sg = padded[rank * per:(rank + 1) * per].clone()
                        st = _unwrap(p.shard)
                        st.grad = sg if st.grad is None else st.grad + sg
                        return g
                    return hook
                t.register_hook(make_hook())
                t.data = torch.empty(0, dtype=t.dtype, device=t.device)

            def pre(m, x, state=state):
                for p, shape in state:
                    _unwrap(p).data = _gather_full(_unwrap(p.shard), shape, world).clone()
                return None

            def post(m, x, out, state=state):
                o = _unwrap(out)
                if o.requires_grad:
                    def regather(_g, state=state):
                        for p, shape in state:
                            if _unwrap(p).numel() == 0:
                                _unwrap(p).data = _gather_full(_unwrap(p.shard), shape, world).clone()
                        return None
                    o.register_hook(regather)
                return None
            leaf.register_forward_pre_hook(pre)
            leaf.register_forward_hook(post)
        return module

    @staticmethod
    def shards(module) -> List[Tensor]:
        return [p.shard for p in module.parameters() if hasattr(p, "shard")]
