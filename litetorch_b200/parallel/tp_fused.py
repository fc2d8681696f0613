"""Fused tensor-parallel / sequence-parallel linears on symmetric memory.

`TPFusedContext.ag_linear(x_shard, w, b)`:   y = all_gather(x_shard) @ w^T + b   - the all-gather runs inside the
GEMM kernel (`lt_ag_gemm_bf16`, gather CTAs copy the peers' sequence shards while tiles of arrived row blocks
compute); `TPFusedContext.linear_rs(x, w)`:  y_shard = reduce_scatter(x @ w^T)   - the reduce-scatter runs in
the GEMM epilogue and tail (`lt_gemm_rs_bf16`).  Both are autograd functions whose backward uses the mirror-image
fused kernel: d(all-gather -> GEMM) = GEMM -> reduce-scatter and vice versa; weight gradients reuse the gathered
activation that the forward (or the backward's gather) already assembled in local memory.

Attach to layers with `attach(column_layer, row_layer, ctx)`; the layers fall back to NCCL collectives without it.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..ops import kernels as K
from .fsdp import SymmetricBuffer


class TPFusedContext:
    def __init__(self, max_rows: int, max_cols: int, device, group=None, n_comm: int = 0):
        """max_rows: global sequence rows (tokens) of the largest activation; max_cols: its widest feature dimension;
        n_comm: gather CTAs of the all-gather GEMMs (0: chosen per call from the GEMM's FLOPs and the bytes to fetch)."""
        self.group = group or dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.device = torch.device(device)
        self.n_comm = n_comm
        n = max_rows * max_cols
        W = self.world
        # two slots each (parity of the call counter): a rank may start call e+1 while a peer still reads call e
        self.shard = [SymmetricBuffer(n // W, torch.bfloat16, self.device, self.group) for _ in range(2)]
        self.stage = [SymmetricBuffer(n, torch.bfloat16, self.device, self.group) for _ in range(2)]
        self.counters = [SymmetricBuffer(4096, torch.int32, self.device, self.group) for _ in range(2)]
        self.flags = SymmetricBuffer(64 * 8, torch.int32, self.device, self.group)
        self.full = torch.empty(n, dtype=torch.bfloat16, device=self.device)      # gathered activation (local)
        self.gather_flags = torch.zeros(4096, dtype=torch.int32, device=self.device)
        self.ag_calls = 0
        self.rs_calls = [0, 0]
        self.rs_total = 0
        self.barrier_epoch = 0

    # ---- raw fused ops (no autograd)
    def _barrier(self):
        self.barrier_epoch += 1
        K.signal_barrier(self.flags.tensor, self.flags.ptrs, 0, self.barrier_epoch, self.world, self.rank)

    def input_slot(self, rows: int, cols: int) -> torch.Tensor:
        """[rows, cols] view of the symmetric slot the NEXT gather reads this rank's rows from.  A producer that writes
        its result here and passes the view to `gather_gemm` saves the copy into the slot.  The slot alternates with
        every gather; the one returned here was last read by the peers two gathers ago, and the barrier of the gather
        in between has shown that they are done with it."""
        return self.shard[self.ag_calls & 1].tensor[:rows * cols].view(rows, cols)

    def gather_gemm(self, x_shard: torch.Tensor, w: torch.Tensor, bias=None, b_major: int = 0, full_out: torch.Tensor = None):
        """y = all_gather(x_shard) @ op(w) with the gather inside the GEMM kernel.
        b_major 0: w is [N, K] (y = x @ w^T); 1: w is [K, N] (y = x @ w).
        Returns (y [M, N], x_full [M, K]).  x_full is `full_out` when given (a local [M, K] tensor the caller keeps),
        else a view of the context's own buffer that is only valid until the next gather."""
        rows, Kd = x_shard.shape
        M = rows * self.world
        slot = self.ag_calls & 1
        self.ag_calls += 1
        sh = self.shard[slot].tensor[:rows * Kd].view(rows, Kd)
        if x_shard.data_ptr() != sh.data_ptr():
            sh.copy_(x_shard)
        full = self.full[:M * Kd].view(M, Kd) if full_out is None else full_out
        assert full.shape == (M, Kd) and full.is_contiguous()
        # This rank's own rows need no gather: they go straight into the assembled operand and their chunk flags are
        # set to this call's epoch, so the gather CTAs only fetch the peers' rows and the first tiles start at once.
        full[self.rank * rows:(self.rank + 1) * rows].copy_(x_shard)
        if rows % 128 == 0:
            self.gather_flags[self.rank * rows // 128:(self.rank + 1) * rows // 128].fill_(self.ag_calls)
        self._barrier()                                    # every rank's shard is in place
        if b_major == 0:
            y = K.ag_gemm(None, full, gather_operand=0, shard_ptrs=self.shard[slot].ptrs, world=self.world, rank=self.rank,
                          rows_per_rank=rows, flags=self.gather_flags, epoch=self.ag_calls, other=w, bias=bias,
                          n_comm=self.n_comm)
        else:
            assert bias is None
            y = _ag_gemm_nn(self, full, w, slot, rows)
        return y, full

    def gemm_scatter(self, x: torch.Tensor, w: torch.Tensor, b_major: int = 0, bias=None, residual=None):
        slot = self.rs_total & 1
        self.rs_total += 1
        self.rs_calls[slot] += 1
        return K.gemm_rs(x, w, b_major=b_major, stage_ptrs=self.stage[slot].ptrs, counter_ptrs=self.counters[slot].ptrs,
                         epoch=self.rs_calls[slot], world=self.world, rank=self.rank, bias=bias, residual=residual)

    # ---- autograd wrappers
    def ag_linear(self, x_shard, w, b=None):
        return _AGLinear.apply(self, x_shard, w, b)

    def linear_rs(self, x, w):
        return _LinearRS.apply(self, x, w)


def _flat2(x):
    return x.reshape(-1, x.shape[-1])


class _AGLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, tp, x_shard, w, b):
        x2 = _flat2(x_shard).contiguous()
        y, full = tp.gather_gemm(x2, w.contiguous(), b)
        ctx.tp = tp
        ctx.save_for_backward(full.clone(), w)      # the gathered activation is reused for the weight gradient
        ctx.has_bias = b is not None
        ctx.in_shape = x_shard.shape
        lead = (x_shard.shape[0] * tp.world,) + tuple(x_shard.shape[1:-1])
        return y.view(*lead, w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x_full, w = ctx.saved_tensors
        tp = ctx.tp
        dy2 = _flat2(dy).contiguous()
        dx = tp.gemm_scatter(dy2, w.contiguous(), b_major=1)           # reduce-scatter(dy @ w) over the sequence
        dw = K.gemm(dy2, x_full, a_major=1, b_major=1)
        db = dy2.float().sum(0).to(dy2.dtype) if ctx.has_bias else None
        return None, dx.view(ctx.in_shape), dw, db


class _LinearRS(torch.autograd.Function):
    @staticmethod
    def forward(ctx, tp, x, w):
        x2 = _flat2(x).contiguous()
        y = tp.gemm_scatter(x2, w.contiguous(), b_major=0)
        ctx.tp = tp
        ctx.save_for_backward(x2, w)
        ctx.in_shape = x.shape
        lead = (x.shape[0] // tp.world,) + tuple(x.shape[1:-1])
        return y.view(*lead, w.shape[0])

    @staticmethod
    def backward(ctx, dy_shard):
        x2, w = ctx.saved_tensors
        tp = ctx.tp
        # dx = all_gather(dy) @ w  : gathered inside the GEMM; dw = all_gather(dy)^T @ x from the same gathered buffer
        dyg = _flat2(dy_shard).contiguous()
        rows, N = dyg.shape
        M = rows * tp.world
        slot = tp.ag_calls & 1
        tp.ag_calls += 1
        tp.shard[slot].tensor[:rows * N].view(rows, N).copy_(dyg)
        tp._barrier()
        full = tp.full[:M * N].view(M, N)
        # C[M, K_in] = full[M, N] @ w[N, K_in]  (b stored [K=N, N=K_in] -> b_major 1); gather operand A by M blocks
        dx = _ag_gemm_nn(tp, full, w.contiguous(), slot, rows)
        dw = K.gemm(full, x2, a_major=1, b_major=1)
        return None, dx.view(ctx.in_shape), dw


def _ag_gemm_nn(tp, full, w, slot, rows):
    import ctypes
    from ctypes import c_void_p
    M, N = full.shape
    Kin = w.shape[1]
    out = torch.empty((M, Kin), dtype=torch.bfloat16, device=full.device)
    arr = K._ptr_array(tp.shard[slot].ptrs)
    rc = K._fn("lt_ag_gemm_bf16")(full.data_ptr(), w.data_ptr(), out.data_ptr(), M, Kin, N, full.stride(0), w.stride(0), out.stride(0),
                                  0, 1, 0, None, None, 0, 0, 0, 1.0, 0, ctypes.cast(arr, c_void_p), tp.world, tp.rank, rows,
                                  full.data_ptr(), tp.gather_flags.data_ptr(), tp.ag_calls, tp.n_comm, None, None, 0, K._stream())
    K._check(rc, "lt_ag_gemm_bf16")
    return out


def attach(ctx: TPFusedContext, *layers):
    for l in layers:
        l.fused = ctx
