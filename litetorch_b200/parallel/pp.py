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
        self._sent_shape = False
        self._group_bwd = None
        self.overlap = True

    def _backward_group(self):
        """A second communicator over the same ranks, used only for gradients (stage r+1 -> r).  With activations on one
        communicator and gradients on the other, every communicator carries traffic in one direction only: a send can
        only wait for a receive that its neighbour has already posted, never for one queued behind the neighbour's own
        send, so sends and receives need not be grouped into pairs and a receive can be posted long before its data is
        needed.  Every rank of the job creates every stage group's twin, in the same order (new_group is collective)."""
        if self._group_bwd is None and dist.is_initialized() and self.world > 1:
            mine = tuple(dist.get_process_group_ranks(self.group) if self.group is not None else range(dist.get_world_size()))
            lists = [None] * dist.get_world_size()
            dist.all_gather_object(lists, mine)
            for ranks in sorted(set(tuple(l) for l in lists)):
                g = dist.new_group(list(ranks))
                if ranks == mine:
                    self._group_bwd = g
        return self._group_bwd

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
    def forward(self, input: Optional[Tensor] = None) -> Optional[Tensor]:
        """recv (unless first) -> local module -> send (unless last).  Returns the output on the last stage."""
        x = input
        if not self.is_first and self.world > 1:
            x = Tensor(self._recv_activation(self.rank - 1))
        out = self.local_module(x)
        if not self.is_last and self.world > 1:
            self._send(_unwrap(out).detach(), self.rank + 1, with_shape=not self._sent_shape)
            self._sent_shape = True
            return None
        return out

    __call__ = forward

    def forward_microbatches(self, microbatches: Sequence[Tensor]) -> List[Optional[Tensor]]:
        return [self.forward(mb) for mb in microbatches]

    def schedule_1f1b(self, microbatches: Sequence[Tensor]) -> List[Optional[Tensor]]:
        return self.forward_microbatches(microbatches)

    # ---- training
    def _batched(self, send_t, send_peer, recv_buf, recv_peer):
        """One grouped isend + irecv (either may be None): neighbouring stages post the mirror-image pair, so neither
        side can block the other - which plain send-then-recv orderings do in the 1F1B steady state."""
        ops = []
        if send_t is not None:
            ops.append(dist.P2POp(dist.isend, send_t.contiguous(), self._global(send_peer), self.group))
        if recv_buf is not None:
            ops.append(dist.P2POp(dist.irecv, recv_buf, self._global(recv_peer), self.group))
        if ops:
            for w in dist.batch_isend_irecv(ops):
                w.wait()

    def train_step_1f1b(self, microbatches: Sequence, loss_fn: Callable, targets: Optional[Sequence] = None) -> float:
        """One optimisation step's forward/backward over `microbatches` with the 1F1B schedule.

        On the first stage each micro-batch is the input tensor; on the last stage `loss_fn(output, target_or_mb)`
        produces the loss.  Returns the mean loss on the last stage (0.0 elsewhere).  Gradients accumulate in the
        local module's parameters.  With `self.overlap` (default) the receive of the gradient is posted before the
        forward it will follow and the receive of the next activation before the backward, sends are not waited for
        until the step ends, and a transfer is only waited for where its tensor is consumed; `overlap = False` is the
        grouped send+receive pair that is waited for at once (kept for comparison)."""
        if self.overlap and self.world > 1:
            return self._train_step_1f1b_overlapped(microbatches, loss_fn, targets)
        M, W, r = len(microbatches), self.world, self.rank
        warm = min(M, W - r - 1)
        steady = M - warm
        fifo = deque()
        total = None                      # sum of the micro-batch losses, kept on the device until the step's end
        first, last = (r == 0 or W == 1), (r == W - 1)

        def run_fwd(i, xin):
            out = _unwrap(self.local_module(Tensor(xin)))
            fifo.append((xin, out, i))
            return out

        def run_bwd(grad_out):
            nonlocal total
            xin, out, i = fifo.popleft()
            if last:
                tgt = targets[i] if targets is not None else microbatches[i]
                loss = _unwrap(loss_fn(Tensor(out), tgt))
                total = loss.detach().float() if total is None else total + loss.detach().float()
                (loss / M).backward()
            else:
                out.backward(grad_out)
            return None if first else xin.grad

        def recv_fwd_plain():
            return self._recv_activation(r - 1).requires_grad_(True)

        def send_fwd_plain(out):
            self._send(out.detach(), r + 1, with_shape=not self._sent_shape)
            self._sent_shape = True

        def new_input(i):
            return _unwrap(microbatches[i]) if first else None

        # warm-up forwards (plain transfers; the first one carries the shape header)
        for i in range(warm):
            xin = new_input(i) if first else recv_fwd_plain()
            out = run_fwd(i, xin)
            if not last:
                send_fwd_plain(out)
        xin = None
        if steady > 0:
            xin = new_input(warm) if first else recv_fwd_plain()
        for k in range(steady):
            i = warm + k
            out = run_fwd(i, xin)
            grad_out = None
            if not last:
                if not self._sent_shape:                     # only possible when warm == 0, i.e. never for a non-last stage
                    send_fwd_plain(out)
                    grad_out = torch.empty_like(out)
                    self._batched(None, 0, grad_out, r + 1)
                else:
                    grad_out = torch.empty_like(out)
                    self._batched(out.detach(), r + 1, grad_out, r + 1)
            gin = run_bwd(grad_out)
            more = k + 1 < steady
            if first:
                xin = new_input(i + 1) if more else None
            else:
                nxt = torch.empty(self._in_shape, dtype=self._in_dtype, device=gin.device) if more else None
                self._batched(gin, r - 1, nxt, r - 1)
                xin = nxt.requires_grad_(True) if more else None
        # drain
        for _ in range(warm):
            grad_out = None
            if not last:
                _, out, _ = fifo[0]
                grad_out = torch.empty_like(out)
                self._batched(None, 0, grad_out, r + 1)
            gin = run_bwd(grad_out)
            if not first:
                self._batched(gin, r - 1, None, 0)
        return float(total) / M if (last and total is not None) else 0.0

    def _train_step_1f1b_overlapped(self, microbatches, loss_fn, targets) -> float:
        M, W, r = len(microbatches), self.world, self.rank
        warm = min(M, W - r - 1)
        steady = M - warm
        first, last = r == 0, r == W - 1
        gf, gb = self.group, self._backward_group()
        fifo = deque()
        sends = []                         # (work, tensor) of sends in flight: waited for once, at the end of the step
        total = None

        def isend(t, peer, group):
            t = t.contiguous()
            sends.append((dist.isend(t, self._global(peer), group=group), t))

        def post_recv_x():
            if first:
                return None
            if self._in_shape is None:     # the first message of a shape carries a header (blocking, once)
                return ("now", self._recv_activation(r - 1))
            buf = torch.empty(self._in_shape, dtype=self._in_dtype, device=self._dev())
            return (dist.irecv(buf, self._global(r - 1), group=gf), buf)

        def take_x(pending, i):
            if first:
                return _unwrap(microbatches[i])
            w, buf = pending
            if w != "now":
                w.wait()
            return buf.requires_grad_(True)

        def run_fwd(i, xin):
            out = _unwrap(self.local_module(Tensor(xin)))
            fifo.append((xin, out, i))
            if not last:
                if not self._sent_shape:
                    self._send(out.detach(), r + 1, with_shape=True)
                    self._sent_shape = True
                else:
                    isend(out.detach(), r + 1, gf)
            return out

        def run_bwd(pending_grad):
            nonlocal total
            xin, out, i = fifo.popleft()
            if last:
                tgt = targets[i] if targets is not None else microbatches[i]
                loss = _unwrap(loss_fn(Tensor(out), tgt))
                total = loss.detach().float() if total is None else total + loss.detach().float()
                (loss / M).backward()
            else:
                w, g = pending_grad
                w.wait()
                out.backward(g)
            if not first:
                isend(xin.grad, r - 1, gb)

        def post_recv_grad(out_like):
            if last:
                return None
            g = torch.empty_like(out_like)
            return (dist.irecv(g, self._global(r + 1), group=gb), g)

        pend_x = post_recv_x()
        for i in range(warm):
            xin = take_x(pend_x, i)
            pend_x = post_recv_x() if i + 1 < M else None      # the next activation travels while this forward runs
            run_fwd(i, xin)
        for k in range(steady):
            i = warm + k
            xin = take_x(pend_x, i)
            # the gradient this stage will need right after the forward: posted now, arrives under the forward
            pend_g = post_recv_grad(fifo[0][1]) if fifo else None
            out = run_fwd(i, xin)
            if pend_g is None:
                pend_g = post_recv_grad(out)
            pend_x = post_recv_x() if i + 1 < M else None      # the next activation arrives under the backward
            run_bwd(pend_g)
        for _ in range(warm):
            run_bwd(post_recv_grad(fifo[0][1]))
        for w, _t in sends:
            w.wait()
        return float(total) / M if (last and total is not None) else 0.0

    run_1f1b_with_backward = train_step_1f1b

    def parameters(self):
        return self.local_module.parameters()

    def to(self, device):
        self.device = device
        self.local_module.to(device)
        return self
