"""Pipeline parallelism: `PipelineParallelModule` with the 1F1B schedule.

Same public methods as the reference (include/litetorch/distributed.h:94-264): `forward`,
`forward_microbatches`, `schedule_1f1b` (forward only), `train_step_1f1b(microbatches, loss_fn)`,
`run_1f1b_with_backward`, `parameters`, `to`.  The schedule is the reference's: `min(M, W - rank - 1)`
warm-up forwards, then one-forward-one-backward, then the drain.  Transport is `torch.distributed` p2p -
NCCL send/recv over NVLink on CUDA (the reference moves activations through host shared memory or TCP:
src/distributed/distributed.cpp:577-748) - with receives for the next step posted before the current
compute so that the transfer overlaps it.  Activation shapes are exchanged once per shape, not per message.
"""
from __future__ import annotations

from collections import deque
from typing import Callable, List, Optional, Sequence

import torch
import torch.distributed as dist

from ..core import Tensor, _unwrap


class PipelineParallelModule:
    def __init__(self, sub_module, group=None, device=None):
        self.local_module = sub_module
        self.group = group
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.device = device
        self._in_shape = None
        self._in_dtype = torch.float32

    # ---- helpers
    def _global(self, r: int) -> int:
        return dist.get_global_rank(self.group, r) if (self.group is not None and dist.is_initialized()) else r

    @property
    def is_first(self) -> bool:
        return self.rank == 0

    @property
    def is_last(self) -> bool:
        return self.rank == self.world - 1

    def _dev(self):
        if self.device is not None:
            return torch.device(self.device)
        if dist.is_initialized() and dist.get_backend() == "nccl":
            return torch.device("cuda", torch.cuda.current_device())
        return torch.device("cpu")

    def _send(self, t: torch.Tensor, dst: int, with_shape: bool):
        t = t.contiguous()
        if with_shape:
            hdr = torch.zeros(10, dtype=torch.int64, device=t.device)
            hdr[0] = t.dim()
            hdr[1] = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}.get(t.dtype, 0)
            hdr[2:2 + t.dim()] = torch.tensor(list(t.shape), device=t.device)
            dist.send(hdr, self._global(dst), group=self.group)
        dist.send(t, self._global(dst), group=self.group)

    def _recv_activation(self, src: int) -> torch.Tensor:
        dev = self._dev()
        if self._in_shape is None:
            hdr = torch.zeros(10, dtype=torch.int64, device=dev)
            dist.recv(hdr, self._global(src), group=self.group)
            h = hdr.tolist()
            self._in_shape = [int(x) for x in h[2:2 + int(h[0])]]
            self._in_dtype = {0: torch.float32, 1: torch.bfloat16, 2: torch.float16}[int(h[1])]
        t = torch.empty(self._in_shape, dtype=self._in_dtype, device=dev)
        dist.recv(t, self._global(src), group=self.group)
        return t

    # ---- forward only
    def forward(self, x: Optional[Tensor] = None) -> Optional[Tensor]:
        """recv (unless first) -> local module -> send (unless last).  Returns the output on the last stage."""
        first_shape = self._in_shape is None
        if not self.is_first and self.world > 1:
            x = Tensor(self._recv_activation(self.rank - 1))
        out = self.local_module(x)
        if not self.is_last and self.world > 1:
            self._send(_unwrap(out).detach(), self.rank + 1, with_shape=first_shape)
            return None if self.world > 1 else out
        return out

    __call__ = forward

    def forward_microbatches(self, microbatches: Sequence[Tensor]) -> List[Optional[Tensor]]:
        return [self.forward(mb) for mb in microbatches]

    def schedule_1f1b(self, microbatches: Sequence[Tensor]) -> List[Optional[Tensor]]:
        return self.forward_microbatches(microbatches)

    # ---- training
    def train_step_1f1b(self, microbatches: Sequence, loss_fn: Callable, targets: Optional[Sequence] = None) -> float:
        """One optimisation step's forward/backward over `microbatches` with the 1F1B schedule.

        On the first stage each micro-batch is the input tensor; on the last stage `loss_fn(output, target_or_mb)`
        produces the loss.  Returns the mean loss on the last stage (0.0 elsewhere).  Gradients accumulate in the
        local module's parameters."""
        M, W, r = len(microbatches), self.world, self.rank
        warm = min(M, W - r - 1)
        fifo = deque()
        total = 0.0
        sent_shape = [False]
        grad_shape_known = [False]

        def fwd(i):
            if r == 0 or W == 1:
                x = _unwrap(microbatches[i])
                xin = x
            else:
                xin = self._recv_activation(r - 1).requires_grad_(True)
            out = _unwrap(self.local_module(Tensor(xin)))
            if r < W - 1:
                self._send(out.detach(), r + 1, with_shape=not sent_shape[0])
                sent_shape[0] = True
            fifo.append((xin, out, i))

        def bwd():
            nonlocal total
            xin, out, i = fifo.popleft()
            if r == W - 1:
                tgt = targets[i] if targets is not None else microbatches[i]
                loss = _unwrap(loss_fn(Tensor(out), tgt))
                total += float(loss.detach())
                (loss / M).backward()
            else:
                g = torch.empty_like(out)
                dist.recv(g, self._global(r + 1), group=self.group)
                out.backward(g)
            if r > 0:
                dist.send(xin.grad.contiguous(), self._global(r - 1), group=self.group)

        for i in range(warm):
            fwd(i)
        for i in range(warm, M):
            fwd(i)
            bwd()
        while fifo:
            bwd()
        return total / M if r == W - 1 else 0.0

    run_1f1b_with_backward = train_step_1f1b

    def parameters(self):
        return self.local_module.parameters()

    def to(self, device):
        self.device = device
        self.local_module.to(device)
        return self
