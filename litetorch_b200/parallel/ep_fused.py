"""Expert-parallel SwiGLU MoE whose dispatch and combine are fused into the grouped expert GEMMs.

Forward:  tokens stay in their rank's symmetric buffer; `lt_moe_gather_gemm` fetches the routed rows from the peers
while the gate/up GEMM of already-arrived slot blocks runs; SwiGLU; `lt_moe_gemm_scatter` multiplies each slot by its
gate weight in the down-projection epilogue and adds it into the owning rank's fp32 output accumulator.
Backward: the same two kernels with the roles swapped (gather dY rows -> dH, scatter-add dX rows), per-expert tcgen05
weight-gradient GEMMs on the saved slot buffers, and the router gradient returned to the source ranks.
Routing metadata (a few bytes per slot) is exchanged with one NCCL all-gather per pass; no payload all-to-all exists.
Requires equal token counts per rank.  Router, capacity factor and auxiliary loss are those of `MoEFeedForward`.
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist

from ..core import Tensor, _unwrap
from ..ops import kernels as K
from .ep import MoEFeedForward
from .fsdp import SymmetricBuffer
from ..utils.sections import section


class MoEFusedFeedForward(MoEFeedForward):
    def __init__(self, dim, ffn, num_experts, top_k=2, capacity_factor=1.25, aux_loss_coef=0.01, group=None, device="cuda",
                 seed=0, init_std=0.02, max_tokens=8192, n_comm=8):
        super().__init__(dim, ffn, num_experts, top_k, capacity_factor, aux_loss_coef, group, torch.bfloat16, device, seed, init_std)
        self.group = group or dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        dev = torch.device(device)
        self.max_tokens = max_tokens
        self.tok = SymmetricBuffer(max_tokens * dim, torch.bfloat16, dev, self.group)      # x (forward) / dy (backward)
        self.acc = SymmetricBuffer(max_tokens * dim, torch.float32, dev, self.group)       # y (forward) / dx (backward)
        self.sig = SymmetricBuffer(64, torch.int32, dev, self.group)
        cap_slots = int(math.ceil(capacity_factor * max_tokens * top_k * self.world / num_experts)) * self.local_E
        self.max_slots = (cap_slots // 128 + self.local_E + 1) * 128
        self.slot_buf = torch.zeros(self.max_slots * dim, dtype=torch.bfloat16, device=dev)
        self.flags = torch.zeros(4096, dtype=torch.int32, device=dev)
        self.epoch = 0
        self.sig_epoch = 0
        self.n_comm = n_comm

    def barrier(self):
        self.sig_epoch += 1
        K.signal_barrier(self.sig.tensor, self.sig.ptrs, 0, self.sig_epoch, self.world, self.rank)

    def _build_slots(self, top_w, top_i, keep):
        """All ranks share (expert, source row, weight) of every kept slot; this rank keeps those of its experts,
        grouped by expert and padded to blocks of 128."""
        N, k = top_i.shape
        dev = top_i.device
        exp = torch.where(keep, top_i, torch.full_like(top_i, -1)).reshape(-1)
        meta = torch.stack([exp.float(), torch.arange(N, device=dev).repeat_interleave(k).float(), top_w.detach().reshape(-1).float()], 1)
        allm = [torch.empty_like(meta) for _ in range(self.world)]
        dist.all_gather(allm, meta.contiguous(), group=self.group)
        allm = torch.stack(allm, 0)                                        # [W, N*k, 3]
        e = allm[:, :, 0].long()
        NK = e.shape[1]
        mine = (e >= self.first) & (e < self.first + self.local_E)
        # local expert of every slot of every rank, `local_E` for slots routed elsewhere (they sort last)
        le_all = torch.where(mine, e - self.first, torch.full_like(e, self.local_E)).reshape(-1)
        counts_cpu = torch.bincount(le_all, minlength=self.local_E + 1)[:self.local_E].tolist()   # the layer's one host sync
        n_mine = sum(counts_cpu)
        order = torch.argsort(le_all, stable=True)[:n_mine]        # grouped by expert, (source rank, slot) order inside
        src_rank, flat, le = order // NK, order % NK, le_all[order]
        padded_cpu = [(c + 127) // 128 * 128 for c in counts_cpu]
        starts_cpu, excl_cpu, acc_p, acc_c = [], [], 0, 0
        for c, pc in zip(counts_cpu, padded_cpu):
            starts_cpu.append(acc_p)
            excl_cpu.append(acc_c)
            acc_p += pc
            acc_c += c
        S = max(acc_p, 128)
        assert S <= self.max_slots, "more routed tokens than the slot buffer holds"
        starts = torch.tensor(starts_cpu, dtype=torch.int64, device=dev)
        excl = torch.tensor(excl_cpu, dtype=torch.int64, device=dev)
        pos = starts[le] + (torch.arange(n_mine, device=dev) - excl[le])
        slot = torch.full((S, 2), -1, dtype=torch.int32, device=dev)
        slot[pos, 0] = src_rank.int()
        slot[pos, 1] = allm[src_rank, flat, 1].int()
        w = torch.zeros(S, dtype=torch.float32, device=dev)
        w[pos] = allm[src_rank, flat, 2]
        origin = torch.full((S, 2), -1, dtype=torch.int64, device=dev)    # (source rank, flat slot index n*k+j)
        origin[pos, 0] = src_rank
        origin[pos, 1] = flat
        # expert of every 128-row block: the first expert whose padded range ends beyond the block's first row
        ends_cpu = [st + pc for st, pc in zip(starts_cpu, padded_cpu)]
        group_cpu = [min(sum(1 for en in ends_cpu if en <= b * 128), self.local_E - 1) for b in range(S // 128)]
        group = torch.tensor(group_cpu, dtype=torch.int32, device=dev)
        self._group_cpu = group_cpu
        return slot.contiguous(), w, group.contiguous(), origin, S

    def forward(self, x: Tensor) -> Tensor:
        xt = _unwrap(x)
        shape = xt.shape
        x2 = xt.reshape(-1, shape[-1])
        with section("moe.route"):
            top_w, top_i, keep, aux = self.route(x2)
        self.last_aux_loss = aux * self.aux_loss_coef
        self._dropped = (~keep).sum()                 # read lazily: no host sync in the step
        y = _MoEFused.apply(self, x2, top_w, top_i, keep, _unwrap(self.w_gate_up), _unwrap(self.w_down))
        return Tensor(y.view(shape))

    __call__ = forward


class _MoEFused(torch.autograd.Function):
    @staticmethod
    def forward(ctx, m, x2, top_w, top_i, keep, w_gu, w_dn):
        N, d = x2.shape
        with section("moe.fwd.build_slots"):
            slot, w, group, origin, S = m._build_slots(top_w, top_i, keep)
        tok = m.tok.tensor[:N * d].view(N, d)
        acc = m.acc.tensor[:N * d].view(N, d)
        with section("moe.fwd.publish"):
            m.barrier()                                   # peers are done with the previous contents of tok / acc
            tok.copy_(x2)
            acc.zero_()
            m.barrier()                                   # tokens published, accumulators cleared
        m.epoch += 1
        sb = m.slot_buf[:S * d].view(S, d)
        with section("moe.fwd.gather_gemm"):
            gu = K.moe_gather_gemm(m.tok.ptrs, m.world, slot, group, w_gu, b_major=0, slot_buf=sb, flags=m.flags, epoch=m.epoch,
                                   n_comm=m.n_comm)
        # Padding slots (the tail of every expert's last 128-row block) carry no token: the gather fills their rows of
        # the staging buffer from a row of zeros.  Nothing reads them in the forward (the combine skips them), but the
        # weight-gradient GEMMs sum over all rows of a block, so the saved copy of the routed inputs is cleared there
        # once more (masked, not multiplied: 0 * NaN is NaN); the rows of gu need no clearing, the backward's pointwise
        # kernel never reads them.
        with section("moe.fwd.pointwise"):
            pad = (slot[:, 0] < 0)[:, None]
            xs = sb.clone().masked_fill_(pad, 0)          # routed inputs, kept for the weight gradient
            h = K.swiglu_fwd(gu)
        with section("moe.fwd.gemm_scatter"):
            K.moe_gemm_scatter(h, group, w_dn, b_major=0, slot_dst=slot, row_weight=w, acc_ptrs=m.acc.ptrs, world=m.world)
            m.barrier()                                   # every rank has added its experts' outputs
            y = acc.to(torch.bfloat16)
        ctx.m = m
        ctx.group_cpu = m._group_cpu
        ctx.save_for_backward(slot, w, group, origin, xs, gu, w_gu, w_dn)
        ctx.meta = (N, d, S, top_w.shape)
        return y

    @staticmethod
    def backward(ctx, dy):
        m = ctx.m
        slot, w, group, origin, xs, gu, w_gu, w_dn = ctx.saved_tensors
        N, d, S, tw_shape = ctx.meta
        tok = m.tok.tensor[:N * d].view(N, d)
        acc = m.acc.tensor[:N * d].view(N, d)
        with section("moe.bwd.publish"):
            m.barrier()
            tok.copy_(dy)
            acc.zero_()
            m.barrier()
        m.epoch += 1
        sb = m.slot_buf[:S * d].view(S, d)
        # dh (unweighted) = dy_slot @ W_down : gather dy rows, B stored [E, K=d, N=F]
        with section("moe.bwd.gather_gemm"):
            dh_u = K.moe_gather_gemm(m.tok.ptrs, m.world, slot, group, w_dn, b_major=1, slot_buf=sb, flags=m.flags, epoch=m.epoch,
                                     n_comm=m.n_comm)
        with section("moe.bwd.pointwise"):
            pad = (slot[:, 0] < 0)[:, None]
            dys = sb.masked_fill(pad, 0)                   # gathered dy rows (padding rows cleared, see forward)
            # gate-weight gradient, weighted h and SwiGLU backward in one pass over the slot rows; padding rows come out 0
            dgu, hw, dw_slot = K.moe_expert_bwd(gu, dh_u.contiguous(), w.contiguous(), slot)
        # weight gradients per expert on its slot range
        with section("moe.bwd.wgrad"):
            dwgu, dwdn = torch.zeros_like(w_gu), torch.zeros_like(w_dn)
            g_cpu = ctx.group_cpu
            b0 = 0
            while b0 < len(g_cpu):
                e = g_cpu[b0]
                b1 = b0
                while b1 < len(g_cpu) and g_cpu[b1] == e:
                    b1 += 1
                r0, r1 = b0 * 128, b1 * 128
                K.gemm(dgu[r0:r1], xs[r0:r1], a_major=1, b_major=1, out=dwgu[e], accumulate=True)
                K.gemm(dys[r0:r1], hw[r0:r1], a_major=1, b_major=1, out=dwdn[e], accumulate=True)
                b0 = b1
        # dx: scatter-add dgu_slot @ W_gu into the token owners' accumulators (B stored [E, K=2F, N=d])
        with section("moe.bwd.gemm_scatter"):
            K.moe_gemm_scatter(dgu, group, w_gu, b_major=1, slot_dst=slot, row_weight=None, acc_ptrs=m.acc.ptrs, world=m.world)
        # router gradient: each slot's d(loss)/d(gate weight) goes back to the rank and slot it came from
        with section("moe.bwd.router_grad"):
            send = torch.stack([origin[:, 0].float(), origin[:, 1].float(), dw_slot], 1)
            pad = torch.full((m.max_slots, 3), -1.0, device=send.device)
            pad[:S] = send
            allg = [torch.empty_like(pad) for _ in range(m.world)]
            dist.all_gather(allg, pad, group=m.group)
            allg = torch.cat(allg, 0)
            mine = allg[:, 0].long() == m.rank
            dtw = torch.zeros(tw_shape[0] * tw_shape[1], dtype=torch.float32, device=send.device)
            dtw[allg[mine, 1].long()] = allg[mine, 2]
            m.barrier()
            dx = acc.to(torch.bfloat16)
        return None, dx, dtw.view(tw_shape), None, None, dwgu, dwdn
