"""Llama-style decoder assembled from the parallel building blocks: tensor parallel with sequence parallelism
(all-gather -> GEMM and GEMM -> reduce-scatter fused kernels), context parallel ring FlashAttention, expert-parallel
SwiGLU MoE (dispatch / combine fused into the grouped GEMMs) and pipeline stages.  It covers the model families the
reference builds from `ColumnParallelLinear` / `RowParallelLinear` (src/nn/parallel_linear.cpp:16-132), `MoELinear`
(src/nn/moe.cpp:11-278), `Ops::ring_attention` (src/ops/ring_attention.cpp:13-129) and `PipelineParallelModule`
(src/distributed/pipeline_parallel.cpp:16-115); those pieces are never combined into one model there.

Activations travel as rows [tokens, d_model]: with sequence parallelism every tensor-parallel rank holds a
contiguous slice of the rows of its (context-parallel) token shard.  Parameters are torch tensors that require
grad; `reduce_groups` on a parameter lists the process groups over which its gradient is summed after backward
(replicas across data / context parallel ranks, and row-sliced partial sums of norm gains and embeddings across the
tensor-parallel group).

On CUDA with NCCL the fused contexts are used; without them (CPU, gloo) the same model runs on plain collectives, which
is what the CPU tests exercise.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, replace
from typing import List, Optional

import torch
import torch.distributed as dist

from ..ops import functional as Fn
from ..utils.sections import section
from ..parallel import tp as _tp


@dataclass
class DecoderConfig:
    name: str
    vocab: int
    n_layers: int
    d_model: int
    n_q: int
    n_kv: int
    head_dim: int
    ffn: int
    rope_theta: float = 1e4
    eps: float = 1e-5
    n_experts: int = 0          # 0 = dense SwiGLU MLP
    top_k: int = 2
    capacity_factor: float = 1.25
    aux_coef: float = 0.01

    def n_params(self) -> int:
        attn = self.d_model * (self.n_q + 2 * self.n_kv) * self.head_dim + self.n_q * self.head_dim * self.d_model
        mlp = 3 * self.d_model * self.ffn * max(1, self.n_experts)
        return self.n_layers * (attn + mlp + 2 * self.d_model) + 2 * self.vocab * self.d_model + self.d_model


PRESETS = {
    # tensor parallel 8 with sequence parallelism, seq 8192, 8 sequences per step
    "llama3-8b": DecoderConfig("llama3-8b", 128256, 32, 4096, 32, 8, 128, 14336, rope_theta=5e5),
    # expert parallel 8, data-parallel attention, seq 4096, micro-batch 2 per GPU
    "moe-8x2b": DecoderConfig("moe-8x2b", 32000, 16, 2048, 16, 4, 128, 5632, n_experts=8, top_k=2),
    # TP2 x CP2 x PP2, seq 32768 (zigzag), 8 micro-batches of one sequence, activation checkpointing
    "llama-3b-long": DecoderConfig("llama-3b-long", 32000, 28, 3072, 24, 8, 128, 8192),
    # small shapes with the same structure for tests
    "tiny-dense": DecoderConfig("tiny-dense", 512, 2, 256, 4, 2, 64, 512),
    "tiny-moe": DecoderConfig("tiny-moe", 512, 2, 256, 4, 2, 64, 256, n_experts=4, top_k=2),
}


def _w(group) -> int:
    return dist.get_world_size(group) if (group is not None and dist.is_initialized()) else 1


def _r(group) -> int:
    return dist.get_rank(group) if (group is not None and dist.is_initialized()) else 0


class ParallelDims:
    """Process groups of one rank: tensor (tp), context (cp), expert (ep), data (dp) and pipeline (pp) parallel.
    `None` means that axis has size one.  `tp_fused` / `cp_fused` are the symmetric-memory contexts of the fused
    kernels (None: plain collectives)."""

    def __init__(self, tp=None, cp=None, ep=None, dp=None, pp=None, tp_fused=None, cp_fused=None, zigzag=True, fp8=False,
                 cp_mode="ring"):
        self.tp, self.cp, self.ep, self.dp, self.pp = tp, cp, ep, dp, pp
        self.tp_fused, self.cp_fused, self.zigzag = tp_fused, cp_fused, zigzag
        # "ring": KV blocks of all context-parallel ranks walked by the attention kernels (zigzag split);
        # "ulysses": sequence <-> head all-to-all around a local full-sequence attention (contiguous split)
        assert cp_mode in ("ring", "ulysses")
        self.cp_mode = cp_mode
        if cp_mode == "ulysses":
            self.zigzag = False
        self.fp8 = fp8      # e4m3 GEMMs (1x128 / 128x128 block scales) in the parallel linears; collectives stay NCCL

    @property
    def tp_world(self): return _w(self.tp)
    @property
    def tp_rank(self): return _r(self.tp)
    @property
    def cp_world(self): return _w(self.cp)
    @property
    def cp_rank(self): return _r(self.cp)


# ------------------------------------------------------------------------------------------------ parallel linears
def ag_linear(dims: ParallelDims, x_rows: torch.Tensor, w_local: torch.Tensor) -> torch.Tensor:
    """y = all_gather_rows(x) @ w_local^T   (column-parallel weight, sequence-parallel input)."""
    lin = Fn.linear_fp8 if dims.fp8 else Fn.linear
    if dims.tp_world == 1:
        return lin(x_rows, w_local)
    if dims.tp_fused is not None and not dims.fp8:
        return dims.tp_fused.ag_linear(x_rows, w_local, None)
    full = _tp._GatherFwdScatterBwd.apply(x_rows, 0, dims.tp, True)
    return lin(full, w_local)


def linear_rs(dims: ParallelDims, x: torch.Tensor, w_local: torch.Tensor) -> torch.Tensor:
    """y_rows = reduce_scatter_rows(x @ w_local^T)   (row-parallel weight, sequence-parallel output)."""
    lin = Fn.linear_fp8 if dims.fp8 else Fn.linear
    if dims.tp_world == 1:
        return lin(x, w_local)
    if dims.tp_fused is not None and not dims.fp8:
        return dims.tp_fused.linear_rs(x, w_local)
    return _tp._ScatterFwdGatherBwd.apply(lin(x, w_local), 0, dims.tp)


def _units(units, unit_shape, cat_dim, std, key, device, dtype, reduce_groups=()):
    """A parameter assembled from independently seeded units (a head, a block of feed-forward or vocabulary rows).
    A tensor-parallel rank draws exactly the units it owns, so the same seed gives the same model under every layout:
    the shards of a tensor-parallel group, put side by side, are the tensor one rank alone would draw."""
    parts = []
    for u in units:
        g = torch.Generator().manual_seed((key * 1000003 + int(u)) % (2 ** 62))
        parts.append(torch.empty(*unit_shape).normal_(0, std, generator=g))
    t = torch.cat(parts, cat_dim).to(device=device, dtype=dtype).requires_grad_(True)
    t.reduce_groups = [g for g in reduce_groups if g is not None]
    return t


def _unit_rows(n: int) -> int:
    """Rows per unit of a dimension that tensor parallelism may split up to eight ways."""
    return math.gcd(n // 8, 64) if n % 8 == 0 else 1


def _ones(n, device, dtype, reduce_groups=()):
    t = torch.ones(n, device=device, dtype=dtype).requires_grad_(True)
    t.reduce_groups = [g for g in reduce_groups if g is not None]
    return t


class DecoderBlock:
    def __init__(self, cfg: DecoderConfig, dims: ParallelDims, layer_idx: int, device, dtype, seed: int, max_tokens: int):
        self.cfg, self.dims = cfg, dims
        Wt, rt = dims.tp_world, dims.tp_rank
        assert cfg.n_q % Wt == 0 and cfg.n_kv % Wt == 0 and cfg.ffn % Wt == 0
        self.hq, self.hkv = cfg.n_q // Wt, cfg.n_kv // Wt
        D, d = cfg.head_dim, cfg.d_model
        # weights are drawn unit by unit (see _units): a rank draws the heads / feed-forward rows it owns
        key = lambda tensor_id: (seed * 1009 + layer_idx + 1) * 16 + tensor_id      # noqa: E731
        rep = (dims.cp, dims.dp)                     # replicas of a tensor-parallel shard
        rep_all = (dims.cp, dims.dp, dims.tp)        # replicated everywhere; row-sliced activations give partial sums
        self.norm1 = _ones(d, device, dtype, rep_all)
        self.norm2 = _ones(d, device, dtype, rep_all)
        q_heads = range(rt * self.hq, (rt + 1) * self.hq)
        kv_heads = range(rt * self.hkv, (rt + 1) * self.hkv)
        with torch.no_grad():
            qkv = torch.cat([_units(q_heads, (D, d), 0, 0.02, key(0), "cpu", torch.float32),
                             _units(kv_heads, (D, d), 0, 0.02, key(1), "cpu", torch.float32),
                             _units(kv_heads, (D, d), 0, 0.02, key(2), "cpu", torch.float32)], 0)
        self.wqkv = qkv.to(device=device, dtype=dtype).requires_grad_(True)        # [q heads | k heads | v heads] of this rank
        self.wqkv.reduce_groups = [g for g in rep if g is not None]
        self.wo = _units(q_heads, (d, D), 1, 0.02, key(3), device, dtype, rep)
        self.moe = None
        if cfg.n_experts > 0:
            assert Wt == 1, "the MoE block uses data-parallel attention (no tensor parallelism)"
            if device != "cpu" and torch.device(device).type == "cuda" and dims.ep is not None:
                from ..parallel.ep_fused import MoEFusedFeedForward
                self.moe = MoEFusedFeedForward(d, cfg.ffn, cfg.n_experts, cfg.top_k, cfg.capacity_factor, cfg.aux_coef,
                                               group=dims.ep, device=device, seed=seed * 7919 + layer_idx,
                                               max_tokens=max_tokens)
            else:
                from ..parallel.ep import MoEFeedForward
                self.moe = MoEFeedForward(d, cfg.ffn, cfg.n_experts, cfg.top_k, cfg.capacity_factor, cfg.aux_coef,
                                          group=dims.ep, dtype=dtype, device=device, seed=seed * 7919 + layer_idx)
            from ..core import _unwrap
            gate = _unwrap(self.moe.gate_weight)
            gate.reduce_groups = [g for g in (dims.ep, dims.dp) if g is not None]     # the router is replicated
            for t in (_unwrap(self.moe.w_gate_up), _unwrap(self.moe.w_down)):
                t.reduce_groups = [g for g in (dims.dp,) if g is not None]            # experts live on one EP rank
                # an expert sees tokens of every EP rank, each weighted by that rank's own mean loss
                t.grad_scale = 1.0 / _w(dims.ep)
        else:
            F = cfg.ffn // Wt
            ch = _unit_rows(cfg.ffn)
            assert F % ch == 0
            chunks = range(rt * F // ch, (rt + 1) * F // ch)
            with torch.no_grad():
                gu = torch.cat([_units(chunks, (ch, d), 0, 0.02, key(4), "cpu", torch.float32),
                                _units(chunks, (ch, d), 0, 0.02, key(5), "cpu", torch.float32)], 0)
            self.w_gu = gu.to(device=device, dtype=dtype).requires_grad_(True)       # [gate slice | up slice]
            self.w_gu.reduce_groups = [g for g in rep if g is not None]
            self.w_dn = _units(chunks, (d, ch), 1, 0.02, key(6), device, dtype, rep)

    def parameters(self) -> List[torch.Tensor]:
        ps = [self.norm1, self.norm2, self.wqkv, self.wo]
        if self.moe is not None:
            from ..core import _unwrap
            ps += [_unwrap(p) for p in self.moe.parameters()]
        else:
            ps += [self.w_gu, self.w_dn]
        return ps

    def forward(self, x_rows: torch.Tensor, B: int, T_local: int, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
        cfg, dims = self.cfg, self.dims
        D = cfg.head_dim
        with section("blk.fwd.qkv_rope"):
            h = Fn.rms_norm(x_rows, self.norm1, cfg.eps)
            qkv = ag_linear(dims, h, self.wqkv).view(B, T_local, self.hq + 2 * self.hkv, D)
            q, k, v = qkv[:, :, :self.hq], qkv[:, :, self.hq:self.hq + self.hkv], qkv[:, :, self.hq + self.hkv:]
            q = Fn.rope_bthd(q, cos, sin).contiguous()
            k = Fn.rope_bthd(k, cos, sin).contiguous()
            v = v.contiguous()
        with section("blk.fwd.attention"):
            if dims.cp_world > 1 and dims.cp_mode == "ulysses":
                from ..parallel.ulysses import ulysses_attention
                a = ulysses_attention(q, k, v, dims.cp, causal=True)
            elif dims.cp_world > 1:
                if dims.cp_fused is not None:
                    a = dims.cp_fused.attention(q, k, v, causal=True)
                else:
                    from ..parallel.cp import ring_attention
                    a = ring_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), dims.cp, causal=True,
                                       zigzag=dims.zigzag).transpose(1, 2)
            else:
                a = Fn.flash_attention_bthd(q, k, v, causal=True)
        with section("blk.fwd.attn_out"):
            a = a.reshape(B * T_local, self.hq * D)
            x_rows = x_rows + linear_rs(dims, a, self.wo)
            h = Fn.rms_norm(x_rows, self.norm2, cfg.eps)
        if self.moe is not None:
            from ..core import Tensor, _unwrap
            with section("blk.fwd.moe"):
                y = _unwrap(self.moe.forward(Tensor(h)))
            self.aux_loss = self.moe.last_aux_loss
            return x_rows + y
        with section("blk.fwd.ffn"):
            gu = ag_linear(dims, h, self.w_gu)
            return x_rows + linear_rs(dims, Fn.swiglu(gu), self.w_dn)


class ParallelDecoder:
    """Layers [first_layer, last_layer) of the decoder on this pipeline stage, with the embedding on the first stage
    and the final norm, the vocabulary-parallel LM head and the loss on the last."""

    def __init__(self, cfg: DecoderConfig, dims: ParallelDims, device="cuda", dtype=torch.bfloat16, seed: int = 0,
                 first_layer: int = 0, last_layer: Optional[int] = None, max_tokens: int = 8192,
                 activation_checkpointing: bool = False):
        self.cfg, self.dims, self.device, self.dtype = cfg, dims, device, dtype
        last_layer = cfg.n_layers if last_layer is None else last_layer
        self.is_first, self.is_last = first_layer == 0, last_layer == cfg.n_layers
        self.ckpt = activation_checkpointing
        self.blocks = [DecoderBlock(cfg, dims, i, device, dtype, seed, max_tokens) for i in range(first_layer, last_layer)]
        rep_all = (dims.cp, dims.dp, dims.tp)
        vch = _unit_rows(cfg.vocab)
        mkey = lambda tensor_id: (seed * 1009) * 16 + tensor_id                      # noqa: E731
        self.embed = (_units(range(cfg.vocab // vch), (vch, cfg.d_model), 0, 0.02, mkey(7), device, dtype, rep_all)
                      if self.is_first else None)
        if self.is_last:
            Wt, rt = dims.tp_world, dims.tp_rank
            assert cfg.vocab % Wt == 0
            self.v_local = cfg.vocab // Wt
            self.v_start = rt * self.v_local
            self.final_norm = _ones(cfg.d_model, device, dtype, rep_all)
            assert self.v_local % vch == 0
            self.head = _units(range(rt * self.v_local // vch, (rt + 1) * self.v_local // vch), (vch, cfg.d_model), 0, 0.02,
                               mkey(8), device, dtype, (dims.cp, dims.dp))
        self._rope_cache = {}

    # ---- parameters and gradient reductions
    def parameters(self) -> List[torch.Tensor]:
        ps = []
        if self.embed is not None:
            ps.append(self.embed)
        for b in self.blocks:
            ps += b.parameters()
        if self.is_last:
            ps += [self.final_norm, self.head]
        return ps

    def reduce_gradients(self):
        """Sum every gradient over the groups its parameter is replicated (or partially summed) on; data- and
        context-parallel replicas are averaged because every rank's loss is a mean over its own tokens."""
        dims = self.dims
        avg = {id(g): _w(g) for g in (dims.cp, dims.dp, dims.ep) if g is not None}
        for p in self.parameters():
            if p.grad is None:
                continue
            if getattr(p, "grad_scale", 1.0) != 1.0:
                p.grad.mul_(p.grad_scale)
            for g in getattr(p, "reduce_groups", ()):
                if _w(g) > 1:
                    dist.all_reduce(p.grad, group=g)
                    if id(g) in avg and g is not dims.tp:
                        p.grad.div_(avg[id(g)])

    # ---- positions
    def _rope(self, T_local: int):
        key = T_local
        if key not in self._rope_cache:
            cfg, dims = self.cfg, self.dims
            if dims.cp_world > 1 and dims.zigzag:
                from ..parallel.cp import zigzag_positions
                pos = zigzag_positions(dims.cp_rank, dims.cp_world, T_local, device=self.device).float()
            else:
                pos = torch.arange(T_local, device=self.device).float() + dims.cp_rank * T_local
            inv = cfg.rope_theta ** (-torch.arange(0, cfg.head_dim, 2, device=self.device).float() / cfg.head_dim)
            ang = pos[:, None] * inv[None, :]
            self._rope_cache[key] = (ang.cos().contiguous(), ang.sin().contiguous())
        return self._rope_cache[key]

    def _row_slice(self, n_rows: int):
        Wt, rt = self.dims.tp_world, self.dims.tp_rank
        assert n_rows % Wt == 0
        return slice(rt * (n_rows // Wt), (rt + 1) * (n_rows // Wt))

    # ---- stages
    def embed_tokens(self, ids: torch.Tensor) -> torch.Tensor:
        """ids [B, T_local] of this context-parallel shard -> the sequence-parallel row slice [B*T_local / tp, d]."""
        flat = ids.reshape(-1)
        return Fn.embedding(flat[self._row_slice(flat.numel())].contiguous(), self.embed)

    def run_layers(self, x_rows: torch.Tensor, B: int, T_local: int) -> torch.Tensor:
        cos, sin = self._rope(T_local)
        for blk in self.blocks:
            if self.ckpt and x_rows.requires_grad:
                x_rows = torch.utils.checkpoint.checkpoint(blk.forward, x_rows, B, T_local, cos, sin, use_reentrant=False)
            else:
                x_rows = blk.forward(x_rows, B, T_local, cos, sin)
        return x_rows

    def loss(self, x_rows: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        """Mean next-token cross entropy over this rank's token shard; targets [B, T_local] (already shifted)."""
        dims = self.dims
        h = Fn.rms_norm(x_rows, self.final_norm, self.cfg.eps)
        logits = ag_linear(dims, h, self.head)                       # [B*T_local, V / tp]
        tgt = targets.reshape(-1)
        if dims.tp_world > 1:
            return _tp.vocab_parallel_cross_entropy(logits, tgt, self.v_start, dims.tp)
        return Fn.cross_entropy(logits, tgt)

    def aux_loss(self):
        terms = [b.aux_loss for b in self.blocks if getattr(b, "aux_loss", None) is not None]
        return sum(terms) if terms else None

    def forward_loss(self, ids: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        """Whole model on one stage: ids, targets [B, T_local]."""
        B, T_local = ids.shape
        x = self.run_layers(self.embed_tokens(ids), B, T_local)
        loss = self.loss(x, targets)
        aux = self.aux_loss()
        return loss if aux is None else loss + aux


def shard_batch(ids: torch.Tensor, dims: ParallelDims) -> torch.Tensor:
    """[B, T] -> this context-parallel rank's tokens [B, T / cp] (zigzag halves when configured)."""
    if dims.cp_world == 1:
        return ids
    if dims.zigzag:
        from ..parallel.cp import zigzag_split
        return zigzag_split(ids, dims.cp_rank, dims.cp_world, dim=1).contiguous()
    return ids.chunk(dims.cp_world, 1)[dims.cp_rank].contiguous()


def tiny(cfg: DecoderConfig, **kw) -> DecoderConfig:
    return replace(cfg, **kw)
