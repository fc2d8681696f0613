"""FSDP (ZeRO-3) x tensor parallelism (+ sequence parallelism) weights for the hand-scheduled Llama engine.

The ranks of one node form a dp x tp mesh (rank = dp_index * tp + tp_index, so a tensor-parallel group sits on
neighbouring GPUs).  Every matrix is first cut the Megatron way over the tp axis - QKV and gate/up by output rows
(whole heads / feed-forward units), attention-output and down projections by input columns, embedding and LM
head by vocabulary rows - and that slice is then sharded by rows over the dp axis together with its fp32 master
copy and AdamW moments (ZeRO-3).  Norm gains are replicated.

Two back-ends implement the same provider interface that `LlamaEngine` schedules against:

* "fused" (CUDA): the tensor-parallel collectives run inside the GEMM kernels over NVLink peer memory
  (`TPFusedContext`: all-gather -> GEMM with gather CTAs, GEMM -> reduce-scatter in the epilogue); the ZeRO-3
  weight all-gather of the next use of a matrix is pulled from the dp peers' shards by `lt_gather_shards` on a
  side stream while the current layer computes (the GEMM's own gather slot is taken by the activation); the
  gradient reduce-scatter is fused with the sharded AdamW update in `lt_rs_adamw`, per layer bucket, under the
  rest of the backward pass; the embedding rows are read straight from the owning rank.
* "collective": the same schedule on `torch.distributed` collectives (gloo on the CPU, NCCL on GPUs) and the
  unfused kernels.  It is what the CPU tests run and what the fused path is compared against.

Reference counterparts: the tp x dp x pp communicator split (src/distributed/distributed.cpp:907-936),
ColumnParallelLinear / RowParallelLinear (src/nn/parallel_linear.cpp:31-106), FSDP::fully_shard
(src/distributed/fsdp_wrapper.cpp:106-156) and ZeRO3Optimizer (src/optim/zero3_optimizer.cpp:11-105).
"""
from __future__ import annotations

import math
import os
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from ..models.llama import LlamaConfig, ParamSpec, kernels_for, param_specs
from .mesh import DeviceMesh

_STAGE_KEYS = ("wqkv", "wo", "w_gu", "w_down", "lm_head")


def _pad128(n: int) -> int:
    return (n + 127) // 128 * 128


def _all_gather_stack(x: torch.Tensor, group, n: int) -> torch.Tensor:
    """[n, *x.shape]: x of every rank of `group`, in rank order."""
    x = x.contiguous()
    out = torch.empty((n * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(out, x, group=group)
    return out.view((n,) + tuple(x.shape))


class TPSlicer:
    """Which rows / columns of every full matrix belong to tensor-parallel rank `t` of `tp`."""

    def __init__(self, cfg: LlamaConfig, tp: int):
        self.cfg, self.tp = cfg, tp
        assert cfg.n_heads % tp == 0 and cfg.n_kv_heads % tp == 0 and cfg.ffn % tp == 0 and cfg.vocab_size % tp == 0

    def local_shape(self, s: ParamSpec) -> Tuple[int, ...]:
        if s.kind == "vector":
            return tuple(s.shape)
        rows, cols = s.shape
        leaf = s.name.split(".")[-1]
        if leaf in ("wo", "w_down"):
            return rows, cols // self.tp
        return rows // self.tp, cols

    def row_index(self, s: ParamSpec, t: int) -> Optional[torch.Tensor]:
        """Rows of the full matrix kept by rank t (None: the matrix is cut by columns instead)."""
        cfg, tp = self.cfg, self.tp
        leaf = s.name.split(".")[-1]
        hd = cfg.head_dim
        if leaf == "wqkv":
            hq, hkv = cfg.n_heads // tp, cfg.n_kv_heads // tp
            q0, k0, v0 = 0, cfg.n_heads * hd, (cfg.n_heads + cfg.n_kv_heads) * hd
            return torch.cat([torch.arange(q0 + t * hq * hd, q0 + (t + 1) * hq * hd),
                              torch.arange(k0 + t * hkv * hd, k0 + (t + 1) * hkv * hd),
                              torch.arange(v0 + t * hkv * hd, v0 + (t + 1) * hkv * hd)])
        if leaf == "w_gu":
            f = cfg.ffn // tp
            return torch.cat([torch.arange(t * f, (t + 1) * f), torch.arange(cfg.ffn + t * f, cfg.ffn + (t + 1) * f)])
        if leaf in ("embed", "lm_head"):
            v = cfg.vocab_size // tp
            return torch.arange(t * v, (t + 1) * v)
        return None

    def take(self, s: ParamSpec, full: torch.Tensor, t: int) -> torch.Tensor:
        if s.kind == "vector" or self.tp == 1:
            return full
        idx = self.row_index(s, t)
        if idx is not None:
            return full.index_select(0, idx.to(full.device))
        c = full.shape[1] // self.tp
        return full[:, t * c:(t + 1) * c]

    def put(self, s: ParamSpec, full: torch.Tensor, part: torch.Tensor, t: int) -> None:
        if s.kind == "vector" or self.tp == 1:
            full.copy_(part)
            return
        idx = self.row_index(s, t)
        if idx is not None:
            full.index_copy_(0, idx.to(full.device), part)
        else:
            c = full.shape[1] // self.tp
            full[:, t * c:(t + 1) * c] = part


class HybridWeights:
    def __init__(self, cfg: LlamaConfig, device, *, tp: int = 1, seed: int = 0, backend: str = "auto",
                 param_dtype=torch.bfloat16, prefetch: bool = True, gather_ctas: int = 64):
        assert dist.is_initialized(), "HybridWeights needs an initialised process group"
        self.cfg = cfg
        self.device = torch.device(device)
        self.K = kernels_for(self.device)
        self.world, self.rank = dist.get_world_size(), dist.get_rank()
        assert self.world % tp == 0, "world size %d is not a multiple of tp %d" % (self.world, tp)
        self.tp, self.dp = tp, self.world // tp
        self.dp_rank, self.tp_rank = divmod(self.rank, tp)
        if backend == "auto":
            backend = "fused" if self.device.type == "cuda" and param_dtype == torch.bfloat16 else "collective"
        assert backend in ("fused", "collective")
        self.backend = backend
        self.fused = backend == "fused"
        self.param_dtype = param_dtype
        self.mesh = DeviceMesh([self.dp, self.tp], "dp tp")
        self.tp_group = self.mesh.get_group("tp") if self.tp > 1 else None
        self.dp_group = self.mesh.get_group("dp") if self.dp > 1 else None
        self.dp_ranks = self.mesh.ranks_along("dp")
        self.tp_ranks = self.mesh.ranks_along("tp")
        self.slicer = TPSlicer(cfg, tp)
        self.vocab_local = cfg.vocab_size // tp
        self.vocab_start = self.tp_rank * self.vocab_local
        self.gather_ctas = int(os.environ.get("LT_HYBRID_GATHER_CTAS", gather_ctas))
        # ---- layouts (elements): TP-slice matrices in a "full" buffer, their dp row shards in a "shard" buffer
        self.specs = param_specs(cfg)
        self.by_name = {s.name: s for s in self.specs}
        self.matrices = [s for s in self.specs if s.kind == "matrix"]
        self.vectors = [s for s in self.specs if s.kind == "vector"]
        self.lshape: Dict[str, Tuple[int, ...]] = {s.name: self.slicer.local_shape(s) for s in self.specs}
        self.full_off: Dict[str, int] = {}
        self.shard_off: Dict[str, int] = {}
        fo = so = 0
        for s in self.matrices:
            rows, cols = self.lshape[s.name]
            assert rows % self.dp == 0, "%s: %d rows do not divide over %d data-parallel ranks" % (s.name, rows, self.dp)
            self.full_off[s.name], self.shard_off[s.name] = fo, so
            fo += _pad128(rows * cols)
            so += _pad128((rows // self.dp) * cols)
        self.n_full, self.n_shard = fo, so
        self.vec_off = {s.name: s.offset for s in self.vectors}
        self.n_vec = max(s.offset + _pad128(math.prod(s.shape)) for s in self.vectors)
        dev, W = self.device, self.world
        # ---- storage
        self._sym = []
        if self.fused and W > 1:
            from .fsdp import SymmetricBuffer
            self.sym_param = SymmetricBuffer(self.n_shard, torch.bfloat16, dev)          # over all ranks: dp gathers + embedding
            self.param_shard = self.sym_param.tensor
            self.n_slots = cfg.n_layers + 4
            self.sym_flags = SymmetricBuffer(self.n_slots * 8, torch.int32, dev)
            if self.dp > 1:
                self.sym_grad = SymmetricBuffer(self.n_full, torch.bfloat16, dev)
                self.grad_full = self.sym_grad.tensor
            else:
                self.sym_grad = None
                self.grad_full = torch.zeros(self.n_full, dtype=torch.bfloat16, device=dev)
            self.flag_epoch = [0] * self.n_slots
            # the dp peers' parameter shards as tensors of this process, for copy-engine gathers (LT_HYBRID_GATHER=kernel
            # keeps the peer-load kernel instead)
            self.peer_param = None
            if self.dp > 1 and os.environ.get("LT_HYBRID_GATHER", "copy") == "copy":
                views = [self.sym_param.peer_tensor(r) for r in self.mesh.ranks_along("dp")]
                if all(v is not None for v in views):
                    self.peer_param = views
        else:
            self.peer_param = None
            self.sym_param = self.sym_grad = self.sym_flags = None
            self.param_shard = torch.zeros(self.n_shard, dtype=param_dtype, device=dev)
            self.grad_full = torch.zeros(self.n_full, dtype=param_dtype, device=dev)
        self.master = torch.zeros(self.n_shard, dtype=torch.float32, device=dev)
        self.m = torch.zeros_like(self.master)
        self.v = torch.zeros_like(self.master)
        self.vec_p = torch.zeros(self.n_vec, dtype=param_dtype, device=dev)
        self.vec_g = torch.zeros(self.n_vec, dtype=param_dtype, device=dev)
        self.vec_master = torch.zeros(self.n_vec, dtype=torch.float32, device=dev)
        self.vec_m = torch.zeros_like(self.vec_master)
        self.vec_v = torch.zeros_like(self.vec_master)
        # ---- init: the same random stream as the single-GPU weights; each rank keeps its tp slice's dp rows
        gen = torch.Generator(device=dev).manual_seed(seed)
        for s in self.specs:
            if s.kind == "matrix":
                full = torch.empty(*s.shape, dtype=torch.float32, device=dev).normal_(0.0, cfg.init_std, generator=gen)
                self._store_master(s, full)
                del full
            else:
                self.vec_master[s.offset:s.offset + math.prod(s.shape)].fill_(1.0)
        self.param_shard.copy_(self.master)
        self.vec_p.copy_(self.vec_master)
        # ---- weight staging for dp > 1: two buffers per kind of matrix (one for the LM head), filled one use ahead
        self.version = 0
        self.stage: Dict[str, List[torch.Tensor]] = {}
        self.resident: Dict[str, List[Optional[tuple]]] = {}
        self.ready: Dict[str, List[Optional[object]]] = {}
        self.last_used: Dict[str, int] = {}
        if self.dp > 1:
            for key in _STAGE_KEYS:
                name = key if key == "lm_head" else "layers.0." + key
                rows, cols = self.lshape[name]
                nbuf = 1 if key == "lm_head" else 2
                self.stage[key] = [torch.empty((rows, cols), dtype=param_dtype, device=dev) for _ in range(nbuf)]
                self.resident[key] = [None] * nbuf
                self.ready[key] = [None] * nbuf
                self.last_used[key] = nbuf - 1
        self.cuda = self.device.type == "cuda"
        self.side = torch.cuda.Stream(device=dev) if self.cuda else None        # reduce-scatter + AdamW
        self.gstream = torch.cuda.Stream(device=dev) if self.cuda else None     # weight gathers
        self.prefetch = prefetch and os.environ.get("LT_HYBRID_PREFETCH", "1") != "0"
        self._trace: List[str] = []
        self._trace_done = False
        self._pos = 0
        self._next_same_key: List[Optional[str]] = []
        self.hyper = None
        self._pending = False
        self.tpctx = None
        # Create every group's communicator now, with a first small collective, rather than inside the first step,
        # where seconds of skew between ranks would meet the bounded waits of the fused kernels.
        for grp in (self.tp_group, self.dp_group, None):
            if grp is not None or self.world > 1:
                dist.all_reduce(torch.zeros(1, device=dev), group=grp)
        if self.cuda:
            torch.cuda.synchronize()
        dist.barrier()

    # ------------------------------------------------------------------ layout helpers
    def _store_master(self, s: ParamSpec, full: torch.Tensor) -> None:
        part = self.slicer.take(s, full, self.tp_rank)
        rows, cols = self.lshape[s.name]
        rpr = rows // self.dp
        mine = part[self.dp_rank * rpr:(self.dp_rank + 1) * rpr].reshape(-1)
        so = self.shard_off[s.name]
        self.master[so:so + mine.numel()].copy_(mine)

    def _stage_key(self, name: str) -> str:
        return name if name in ("lm_head", "embed") else name.split(".")[-1]

    def _dp_ptrs(self, buf, elem_off: int = 0) -> List[int]:
        return [buf.ptrs[r] + elem_off * buf.itemsize for r in self.dp_ranks]

    def shard_view(self, flat: torch.Tensor, name: str) -> torch.Tensor:
        rows, cols = self.lshape[name]
        o = self.shard_off[name]
        return flat[o:o + (rows // self.dp) * cols].view(rows // self.dp, cols)

    def p(self, name: str) -> torch.Tensor:
        s = self.by_name[name]
        assert s.kind == "vector", "matrix parameters are sharded; use the linear providers"
        return self.vec_p[s.offset:s.offset + math.prod(s.shape)]

    def vector_grad(self, name: str) -> torch.Tensor:
        s = self.by_name[name]
        return self.vec_g[s.offset:s.offset + math.prod(s.shape)]

    def g(self, name: str) -> torch.Tensor:
        s = self.by_name[name]
        if s.kind == "vector":
            return self.vector_grad(name)
        o = self.full_off[name]
        rows, cols = self.lshape[name]
        return self.grad_full[o:o + rows * cols].view(rows, cols)

    # ------------------------------------------------------------------ ZeRO-3 weight access
    def _launch_gather(self, name: str, key: str, b: int, after_event) -> None:
        """Fill stage[key][b] with the tp slice of `name` from the dp ranks' shards."""
        dst = self.stage[key][b]
        rows, cols = self.lshape[name]
        n = (rows // self.dp) * cols
        if self.fused:
            with torch.cuda.stream(self.gstream):
                if after_event is not None:
                    self.gstream.wait_event(after_event)
                if self.peer_param is not None:
                    # copy engines: one device-to-device copy per dp rank out of its mapped shard; no SM is involved,
                    # so the transfer runs under whatever kernels the compute stream has resident
                    so = self.shard_off[name]
                    flat = dst.view(-1)
                    for j, peer in enumerate(self.peer_param):
                        flat[j * n:(j + 1) * n].copy_(peer[so:so + n], non_blocking=True)
                else:
                    self.K.gather_shards(self._dp_ptrs(self.sym_param, self.shard_off[name]), [(0, n)], [dst],
                                         max_ctas=self.gather_ctas)
                ev = torch.cuda.Event()
                ev.record(self.gstream)
            self.ready[key][b] = ev
        else:
            dist.all_gather_into_tensor(dst.view(-1), self.shard_view(self.param_shard, name).reshape(-1).contiguous(),
                                        group=self.dp_group)
            self.ready[key][b] = None
        self.resident[key][b] = (name, self.version)

    def _now_event(self):
        if not (self.fused and self.cuda):
            return None
        ev = torch.cuda.Event()
        ev.record()
        return ev

    def weight(self, name: str) -> torch.Tensor:
        """The tp slice of matrix `name`, whole, in local memory (valid until two later uses of the same kind)."""
        if self.dp == 1:
            return self.shard_view(self.param_shard, name)
        key = self._stage_key(name)
        # ---- follow / record the order of uses
        nxt = None
        if self._trace_done:
            if self._pos < len(self._trace) and self._trace[self._pos] == name:
                nxt = self._next_same_key[self._pos]
                self._pos += 1
            else:                       # the order changed (an evaluation pass, another batch shape): start over
                self._trace_done, self._trace, self._pos = False, [name], 0
        else:
            self._trace.append(name)
        bufs = self.stage[key]
        tag = (name, self.version)
        now = None
        hit = [i for i in range(len(bufs)) if self.resident[key][i] == tag]
        if hit:
            b = hit[0]
        else:
            b = (self.last_used[key] + 1) % len(bufs)
            now = self._now_event()
            self._launch_gather(name, key, b, now)
        if self.ready[key][b] is not None:
            torch.cuda.current_stream().wait_event(self.ready[key][b])
        self.last_used[key] = b
        if nxt is not None and self.prefetch and len(bufs) > 1 and (nxt, self.version) not in self.resident[key]:
            self._launch_gather(nxt, key, 1 - b, now or self._now_event())
        return bufs[b]

    # ------------------------------------------------------------------ tensor-parallel linears
    def _tp(self, M: int):
        if self.tpctx is None or self.tpctx_rows < M:
            from .tp_fused import TPFusedContext
            self.tpctx = TPFusedContext(M, self.cfg.d_model, self.device, group=self.tp_group)
            self.tpctx_rows = M
        return self.tpctx

    def _all_gather_rows(self, x: torch.Tensor) -> torch.Tensor:
        out = torch.empty((x.shape[0] * self.tp,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x.contiguous(), group=self.tp_group)
        return out

    def _reduce_scatter_rows(self, y: torch.Tensor) -> torch.Tensor:
        rows = y.shape[0] // self.tp
        if y.is_cuda:
            out = torch.empty((rows,) + tuple(y.shape[1:]), dtype=y.dtype, device=y.device)
            dist.reduce_scatter_tensor(out, y.contiguous(), group=self.tp_group)
            return out
        y = y.clone()
        dist.all_reduce(y, group=self.tp_group)
        return y[self.tp_rank * rows:(self.tp_rank + 1) * rows].contiguous()

    def gather_slot(self, rows, cols):
        """The symmetric-memory slot that the next fused gather will read this rank's rows from: a norm kernel that
        writes its output there saves the copy into the slot (None when nothing is gathered that way)."""
        if self.tp == 1 or not self.fused:
            return None
        return self._tp(rows * self.tp).input_slot(rows, cols)

    def col_linear(self, x, name):
        """(all_gather(x) @ W^T, all_gather(x)): x is this rank's block of token rows, W its slice of output rows."""
        W = self.weight(name)
        if self.tp == 1:
            return self.K.gemm(x, W), x
        if self.fused:
            full = torch.empty((x.shape[0] * self.tp, x.shape[1]), dtype=x.dtype, device=x.device)
            y, full = self._tp(full.shape[0]).gather_gemm(x, W, full_out=full)
            return y, full
        xf = self._all_gather_rows(x)
        return self.K.gemm(xf, W), xf

    def row_linear(self, x, name, residual=None):
        """reduce_scatter(x @ W^T) + residual: x holds this rank's input columns for all rows, W the matching columns."""
        W = self.weight(name)
        if self.tp == 1:
            return self.K.gemm(x, W, residual=residual)
        if self.fused:
            return self._tp(x.shape[0]).gemm_scatter(x, W, b_major=0, residual=residual)
        y = self._reduce_scatter_rows(self.K.gemm(x, W, out_dtype=torch.float32))
        if residual is not None:
            y = y + residual.float()
        return y.to(x.dtype)

    def col_dgrad(self, dy, name):
        """Input gradient of a column-parallel linear: reduce_scatter(dy @ W) over the rows."""
        W = self.weight(name)
        if self.tp == 1:
            return self.K.gemm(dy, W, b_major=1)
        if self.fused:
            return self._tp(dy.shape[0]).gemm_scatter(dy, W, b_major=1)
        return self._reduce_scatter_rows(self.K.gemm(dy, W, b_major=1, out_dtype=torch.float32)).to(dy.dtype)

    def row_dgrad(self, dy, name):
        """Input gradient of a row-parallel linear: (all_gather(dy) @ W, all_gather(dy))."""
        W = self.weight(name)
        if self.tp == 1:
            return self.K.gemm(dy, W, b_major=1), dy
        if self.fused:
            full = torch.empty((dy.shape[0] * self.tp, dy.shape[1]), dtype=dy.dtype, device=dy.device)
            dx, full = self._tp(full.shape[0]).gather_gemm(dy, W, b_major=1, full_out=full)
            return dx, full
        dyf = self._all_gather_rows(dy)
        return self.K.gemm(dyf, W, b_major=1), dyf

    def wgrad(self, dy, x, name, accumulate=False):
        return self.K.gemm(dy, x, a_major=1, b_major=1, out=self.g(name), accumulate=accumulate)

    def reduce_ce_stats(self, stats):
        """Combine (max, sum-exp, target logit) of the vocabulary slices into those of the whole vocabulary."""
        if self.tp == 1:
            return stats
        allst = _all_gather_stack(stats, self.tp_group, self.tp)
        gm = allst[:, :, 0].amax(0)
        gs = (allst[:, :, 1] * torch.exp(allst[:, :, 0] - gm[None])).sum(0)
        gt = allst[:, :, 2].sum(0)
        return torch.stack([gm, gs, gt], 1).contiguous()

    # ------------------------------------------------------------------ embedding
    def embedding(self, tokens):
        """Embedding rows of this rank's block of the token rows ([M / tp, d])."""
        tok = tokens.reshape(-1)
        M = tok.numel()
        rows = M // self.tp
        mine = tok[self.tp_rank * rows:(self.tp_rank + 1) * rows]
        V, D = self.cfg.vocab_size, self.cfg.d_model
        if self.fused and self.world > 1:
            # vocabulary row v lives on tp rank v // (V / tp), and inside that slice on dp rank (v % (V / tp)) // (V / tp / dp)
            owners = [self.sym_param.ptrs[d * self.tp + t] + self.shard_off["embed"] * self.sym_param.itemsize
                      for t in range(self.tp) for d in range(self.dp)]
            return self.K.embedding_fwd_sharded(mine, owners, V, D, V // self.world, self.world)
        if self.dp > 1:
            table = torch.empty(self.lshape["embed"], dtype=self.param_dtype, device=self.device)
            dist.all_gather_into_tensor(table.view(-1), self.shard_view(self.param_shard, "embed").reshape(-1).contiguous(),
                                        group=self.dp_group)
        else:
            table = self.shard_view(self.param_shard, "embed")
        if self.tp == 1:
            return self.K.embedding_fwd(tok, table)
        loc = tok - self.vocab_start
        inside = (loc >= 0) & (loc < self.vocab_local)
        part = self.K.embedding_fwd(loc.clamp(0, self.vocab_local - 1), table) * inside[:, None].to(table.dtype)
        return self._reduce_scatter_rows(part)

    def zero_grad_embed(self):
        self.g("embed").zero_()

    def embedding_backward(self, tokens, dx):
        tok = tokens.reshape(-1)
        if self.tp > 1:
            dx = self._all_gather_rows(dx)
            tok = tok - self.vocab_start            # rows outside this rank's vocabulary slice fall out of range and are skipped
        self.K.embedding_bwd(tok, dx, self.g("embed"))

    # ------------------------------------------------------------------ reduce-scatter + AdamW per bucket
    def begin_step(self, **hyper):
        self.hyper = hyper

    def _bucket_names(self, bucket) -> List[str]:
        if bucket == "head":
            return ["lm_head"]
        if bucket == "embed":
            return ["embed"]
        p = "layers.%d." % bucket
        return [p + k for k in ("wqkv", "wo", "w_gu", "w_down")]

    def _slot(self, bucket) -> int:
        return 1 if bucket == "head" else (2 if bucket == "embed" else 3 + int(bucket))

    def bucket_done(self, bucket):
        """All weight gradients of `bucket` have been issued on the current stream: reduce over dp and update the shard."""
        if self.hyper is None:
            return
        h = self.hyper
        names = self._bucket_names(bucket)
        if self.fused:
            ev = torch.cuda.Event()
            ev.record()
            with torch.cuda.stream(self.side):
                self.side.wait_event(ev)
                if self.dp > 1:
                    slot = self._slot(bucket)
                    self.flag_epoch[slot] += 1
                    segs = []
                    for name in names:
                        rows, cols = self.lshape[name]
                        n = (rows // self.dp) * cols
                        segs.append((self.full_off[name] + self.dp_rank * n, self.shard_off[name], n))
                    self.K.rs_adamw(self._dp_ptrs(self.sym_grad), None, self.master, self.m, self.v, self.param_shard, segs,
                                    lr=h["lr"], beta1=h["beta1"], beta2=h["beta2"], eps=h["eps"], wd=h["weight_decay"],
                                    step=h["step"], my_flags=self.sym_flags.tensor, peer_flag_ptrs=self._dp_ptrs(self.sym_flags),
                                    slot=slot, epoch=self.flag_epoch[slot], world=self.dp, rank=self.dp_rank)
                else:
                    a = self.shard_off[names[0]]
                    b = self.shard_off[names[-1]] + _pad128(math.prod(self.lshape[names[-1]]))
                    self.K.adam_flat(self.master[a:b], self.grad_full[a:b], self.m[a:b], self.v[a:b], self.param_shard[a:b],
                                     lr=h["lr"], beta1=h["beta1"], beta2=h["beta2"], eps=h["eps"], wd=h["weight_decay"],
                                     step=h["step"], adamw=True)
            self._pending = True
            return
        for name in names:
            rows, cols = self.lshape[name]
            g = self.g(name)
            rpr = rows // self.dp
            if self.dp > 1:
                if g.is_cuda:
                    gs = torch.empty((rpr, cols), dtype=g.dtype, device=g.device)
                    dist.reduce_scatter_tensor(gs, g.contiguous(), group=self.dp_group)
                else:
                    gf = g.clone()
                    dist.all_reduce(gf, group=self.dp_group)
                    gs = gf[self.dp_rank * rpr:(self.dp_rank + 1) * rpr]
            else:
                gs = g
            so = self.shard_off[name]
            n = rpr * cols
            self.K.adam_flat(self.master[so:so + n], gs.reshape(-1), self.m[so:so + n], self.v[so:so + n],
                             self.param_shard[so:so + n], lr=h["lr"], beta1=h["beta1"], beta2=h["beta2"], eps=h["eps"],
                             wd=h["weight_decay"], step=h["step"], adamw=True)

    def optimizer_step(self, *, lr, beta1, beta2, eps, weight_decay, step, dyn=None):
        if self.hyper is None:
            # gradients were accumulated without the overlapped path: reduce + update every bucket now
            self.begin_step(lr=lr, beta1=beta1, beta2=beta2, eps=eps, weight_decay=weight_decay, step=step)
            for b in ["head"] + list(reversed(range(self.cfg.n_layers))) + ["embed"]:
                self.bucket_done(b)
        if self.world > 1:
            dist.all_reduce(self.vec_g)        # every rank holds the norm-gain gradient of its own token rows
        self.K.adam_flat(self.vec_master, self.vec_g, self.vec_m, self.vec_v, self.vec_p, lr=lr, beta1=beta1, beta2=beta2,
                         eps=eps, wd=0.0, step=step, adamw=True, dyn=dyn)

    def finish_step(self):
        """Join the side streams and cross a barrier of ALL ranks: the next step reads parameter shards of dp peers
        (weight gathers) and of any rank (embedding rows), so every rank's update must be complete first.  Staged
        weights of this step become stale."""
        if self.fused:
            cur = torch.cuda.current_stream()
            if self._pending:
                cur.wait_stream(self.side)
                self._pending = False
            cur.wait_stream(self.gstream)
            if self.world > 1:
                self.flag_epoch[0] += 1
                self.K.signal_barrier(self.sym_flags.tensor, self.sym_flags.ptrs, 0, self.flag_epoch[0], self.world, self.rank)
        self.version += 1
        if self.dp > 1:
            if self.hyper is not None and not self._trace_done and self._trace:
                # one complete step has been seen: its order of uses is the prefetch schedule
                # for every use: the next matrix of the same kind that differs from the one in use
                nxt: List[Optional[str]] = [None] * len(self._trace)
                later_name: Dict[str, str] = {}
                later_diff: Dict[str, Optional[str]] = {}
                for i in range(len(self._trace) - 1, -1, -1):
                    name = self._trace[i]
                    key = self._stage_key(name)
                    ln = later_name.get(key)
                    if ln is not None:
                        nxt[i] = ln if ln != name else later_diff.get(key)
                    later_diff[key] = nxt[i]
                    later_name[key] = name
                self._next_same_key = nxt
                self._trace_done = True
            if not self._trace_done:
                self._trace = []
            self._pos = 0
        self.hyper = None

    # ------------------------------------------------------------------ whole-model access (checkpoints, tests)
    def gather_full_master(self, name: str) -> torch.Tensor:
        """The whole fp32 master matrix (all tp slices, all dp shards), on every rank."""
        s = self.by_name[name]
        if s.kind == "vector":
            return self.vec_master[s.offset:s.offset + math.prod(s.shape)].clone()
        mine = self.shard_view(self.master, name).contiguous()
        if self.dp > 1:
            part = torch.empty((mine.shape[0] * self.dp, mine.shape[1]), dtype=mine.dtype, device=mine.device)
            dist.all_gather_into_tensor(part, mine, group=self.dp_group)
        else:
            part = mine
        if self.tp == 1:
            return part
        parts = _all_gather_stack(part, self.tp_group, self.tp)
        full = torch.empty(*s.shape, dtype=part.dtype, device=part.device)
        for t in range(self.tp):
            self.slicer.put(s, full, parts[t], t)
        return full

    def gather_full_grad(self, name: str) -> torch.Tensor:
        """The whole gradient of `name` summed over the data-parallel ranks (fp32), on every rank; for tests."""
        s = self.by_name[name]
        if s.kind == "vector":
            g = self.vector_grad(name).float().clone()
            dist.all_reduce(g)
            return g
        g = self.g(name).float().clone()
        if self.dp > 1:
            dist.all_reduce(g, group=self.dp_group)
        if self.tp == 1:
            return g
        parts = _all_gather_stack(g, self.tp_group, self.tp)
        full = torch.empty(*s.shape, dtype=g.dtype, device=g.device)
        for t in range(self.tp):
            self.slicer.put(s, full, parts[t], t)
        return full

    def parameters(self) -> List[torch.Tensor]:
        return [self.gather_full_master(s.name) for s in self.specs]

    def state_tensors(self) -> Dict[str, torch.Tensor]:
        """This rank's shard of the fp32 masters and AdamW moments plus the replicated vectors."""
        return {"master": self.master, "m": self.m, "v": self.v, "vec_master": self.vec_master, "vec_m": self.vec_m,
                "vec_v": self.vec_v}

    def after_load(self) -> None:
        """Rebuild the low-precision shards from the loaded masters; staged weights become stale."""
        self.param_shard.copy_(self.master)
        self.vec_p.copy_(self.vec_master)
        self.version += 1
        if self.cuda:
            torch.cuda.synchronize()
        dist.barrier()

    def load_parameters(self, tensors: List[torch.Tensor]) -> None:
        for s, t in zip(self.specs, tensors):
            t = t.to(self.device, torch.float32).view(*s.shape)
            if s.kind == "matrix":
                self._store_master(s, t)
            else:
                self.vec_master[s.offset:s.offset + math.prod(s.shape)].copy_(t)
        self.param_shard.copy_(self.master)
        self.vec_p.copy_(self.vec_master)
        self.version += 1
