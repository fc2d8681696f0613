"""ZeRO-3 weights for the Llama engine: parameters, fp32 master copies and AdamW states sharded by rows
over the ranks of one node, with the collectives fused into the compute kernels.

* forward / dgrad GEMMs gather their weight from the ranks' shards INSIDE the GEMM kernel
  (`lt_ag_gemm_bf16`: gather CTAs copy peer shards into a local staging buffer chunk by chunk while the
  tcgen05 tiles of already-arrived chunks run);
* weight gradients are written to a symmetric full-size gradient buffer; when a layer's backward is done
  a single kernel on a side stream (`lt_rs_adamw`) signals the peers, waits for their signals, reduces
  this rank's slice over all ranks' buffers through peer loads, applies AdamW to the fp32 master shard and
  writes the bf16 parameter shard - the reduce-scatter, the cast/scale and the optimizer in one pass,
  overlapped with the backward of the next layer;
* norm gains (a few KB) stay replicated; their gradients are all-reduced with NCCL.

The reference's counterparts are `FullyShardedDataParallel` (include/litetorch/fsdp.h:22-130: flat shards,
gather_parameters / shard_parameters), `FSDP::fully_shard` (src/distributed/fsdp_wrapper.cpp:12-156) and
`ZeRO3Optimizer` (src/optim/zero3_optimizer.cpp:11-105: owner updates + broadcast for replicated params).
Symmetric memory and peer pointers come from `torch.distributed._symmetric_memory`; NCCL is used only for
the replicated vectors.
"""
from __future__ import annotations

import math
import os
from typing import Dict, List

import torch
import torch.distributed as dist

from ..models.llama import LlamaConfig, ParamSpec, SingleTPMixin, param_specs
from ..ops import kernels as K


def ensure_process_group():
    if dist.is_initialized():
        return
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29500")
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))


_CANARY_BYTES = 256          # guard area in front of and behind every symmetric buffer
_CANARY_VALUE = 0x5A
_live_buffers = []           # weak references, for check_symmetric_canaries()


def _symm_backend() -> str:
    return os.environ.get("LT_SYMM_BACKEND", "torch")


# CUDA allows an IPC handle to be opened once per process: several buffers that PyTorch placed in one device segment
# share a handle, so mappings are kept here by handle and stay open until the process exits.
_ipc_mappings: Dict[bytes, int] = {}


class SymmetricBuffer:
    """A tensor allocated at the same offset on every rank, with every rank's device pointer to it.

    Two back-ends give the peer pointers: `torch.distributed._symmetric_memory` (default; also offers a multicast
    address) and the native CUDA-IPC path (`LT_SYMM_BACKEND=ipc`: an ordinary device allocation exported with
    `lt_ipc_export`, the handles exchanged through the process group's host-side store, opened on every peer with
    `lt_ipc_open`; no framework-private API involved).

    The allocation carries a 256-byte guard area on both sides filled with a fixed byte; peers write into these buffers
    from inside kernels, and `check()` (or `check_symmetric_canaries()` over all live buffers) tells whether anything
    wrote past either end."""

    def __init__(self, numel: int, dtype, device, group=None):
        import weakref
        import torch.distributed._symmetric_memory as symm_mem
        group = group or dist.group.WORLD
        itemsize = torch.empty((), dtype=dtype).element_size()
        guard = _CANARY_BYTES // itemsize
        ipc = _symm_backend() == "ipc"
        if ipc:
            self._raw = torch.empty(numel + 2 * guard, dtype=dtype, device=device)
        else:
            self._raw = symm_mem.empty(numel + 2 * guard, dtype=dtype, device=device)
        self._raw.zero_()
        self._guards = (self._raw[:guard].view(torch.uint8), self._raw[guard + numel:].view(torch.uint8))
        for g in self._guards:
            g.fill_(_CANARY_VALUE)
        self.tensor = self._raw[guard:guard + numel]
        if ipc:
            self.ptrs = [p + _CANARY_BYTES for p in self._ipc_rendezvous(group)]
            self.mc_ptr = 0
        else:
            self.handle = symm_mem.rendezvous(self._raw, group=group.group_name if hasattr(group, "group_name") else group)
            self.ptrs = [int(p) + _CANARY_BYTES for p in self.handle.buffer_ptrs]
            try:
                self.mc_ptr = (int(self.handle.multicast_ptr) + _CANARY_BYTES
                               if self.handle.has_multicast_support(device.type, device.index) else 0)
            except Exception:
                self.mc_ptr = 0
        self.itemsize = self.tensor.element_size()
        _live_buffers.append(weakref.ref(self))

    def _ipc_rendezvous(self, group) -> List[int]:
        """Export this rank's allocation, exchange (handle, offset) over the group's store, open every peer's."""
        import ctypes
        from .._native import cuda_lib
        lib = cuda_lib()
        lib.lt_ipc_open.restype = ctypes.c_void_p
        torch.cuda.synchronize()
        handle = (ctypes.c_char * 64)()
        off = ctypes.c_ulonglong(0)
        rc = lib.lt_ipc_export(ctypes.c_void_p(self._raw.data_ptr()), handle, ctypes.byref(off))
        if rc != 0:
            raise RuntimeError("lt_ipc_export failed with code %d" % rc)
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        infos = [None] * world
        dist.all_gather_object(infos, (bytes(handle.raw), int(off.value)), group=group)
        ptrs = []
        for r, (h, o) in enumerate(infos):
            if r == rank:
                ptrs.append(self._raw.data_ptr())
                continue
            if h not in _ipc_mappings:
                base, err = ctypes.c_void_p(0), ctypes.c_int(0)
                p = lib.lt_ipc_open(h, ctypes.c_ulonglong(0), ctypes.byref(base), ctypes.byref(err))
                if not p:
                    raise RuntimeError("lt_ipc_open of rank %d's buffer failed with cudaError %d" % (r, err.value))
                _ipc_mappings[h] = int(base.value)
            ptrs.append(_ipc_mappings[h] + o)
        dist.barrier(group=group)
        return ptrs

    def peer_ptrs(self, elem_offset: int = 0) -> List[int]:
        return [p + elem_offset * self.itemsize for p in self.ptrs]

    def peer_tensor(self, rank: int) -> "torch.Tensor | None":
        """Rank `rank`'s copy of this buffer as a tensor of this process (its memory is mapped here), for copies that
        the copy engines can carry (`dst.copy_(buf.peer_tensor(r)[a:b])`); None with the CUDA-IPC back-end."""
        handle = getattr(self, "handle", None)
        if handle is None:
            return None
        guard = _CANARY_BYTES // self.itemsize
        return handle.get_buffer(rank, (self.tensor.numel(),), self.tensor.dtype, guard)

    def check(self) -> bool:
        """True when both guard areas of this rank's copy still hold the canary byte (synchronises the device)."""
        return all(bool((g == _CANARY_VALUE).all()) for g in self._guards)


def check_symmetric_canaries() -> int:
    """Number of live symmetric buffers of this rank whose guard areas were overwritten."""
    bad, keep = 0, []
    for ref in _live_buffers:
        buf = ref()
        if buf is None:
            continue
        keep.append(ref)
        if not buf.check():
            bad += 1
    _live_buffers[:] = keep
    return bad


_STAGE_KEYS = ("wqkv", "wo", "w_gu", "w_down", "lm_head")


class ShardedWeights(SingleTPMixin):
    SLOT_BARRIER = 0

    def __init__(self, cfg: LlamaConfig, device, seed: int = 0, n_comm: int = 8, use_multimem: bool = False):
        ensure_process_group()
        self.cfg = cfg
        self.device = torch.device(device)
        self.world = dist.get_world_size()
        self.rank = dist.get_rank()
        self.n_comm = int(os.environ.get("LT_FSDP_GATHER_CTAS", n_comm))
        W = self.world
        self.specs = param_specs(cfg)
        self.by_name = {s.name: s for s in self.specs}
        self.matrices = [s for s in self.specs if s.kind == "matrix"]
        self.vectors = [s for s in self.specs if s.kind == "vector"]
        # ---- layouts
        self.full_off: Dict[str, int] = {s.name: s.offset for s in self.matrices}
        self.n_full = max(s.offset + (math.prod(s.shape) + 127) // 128 * 128 for s in self.matrices)
        self.shard_off: Dict[str, int] = {}
        off = 0
        for s in self.matrices:
            rows, cols = s.shape
            assert rows % W == 0, "%s: %d rows do not divide over %d ranks" % (s.name, rows, W)
            self.shard_off[s.name] = off
            off += ((rows // W) * cols + 127) // 128 * 128
        self.n_shard = off
        self.vec_off = {s.name: s.offset for s in self.vectors}
        self.n_vec = max(s.offset + (math.prod(s.shape) + 127) // 128 * 128 for s in self.vectors)
        # ---- symmetric memory: parameter shards, full gradients, signal words
        self.sym_param = SymmetricBuffer(self.n_shard, torch.bfloat16, self.device)
        self.sym_grad = SymmetricBuffer(self.n_full, torch.bfloat16, self.device)
        self.n_slots = cfg.n_layers + 4
        self.sym_flags = SymmetricBuffer(self.n_slots * 8, torch.int32, self.device)
        self.use_multimem = bool(use_multimem and self.sym_grad.mc_ptr)
        # ---- local: fp32 master / m / v of the shard, replicated vectors, staging buffers
        self.master = torch.zeros(self.n_shard, dtype=torch.float32, device=self.device)
        self.m = torch.zeros_like(self.master)
        self.v = torch.zeros_like(self.master)
        self.vec_p = torch.zeros(self.n_vec, dtype=torch.bfloat16, device=self.device)
        self.vec_g = torch.zeros(self.n_vec, dtype=torch.bfloat16, device=self.device)
        self.vec_master = torch.zeros(self.n_vec, dtype=torch.float32, device=self.device)
        self.vec_m = torch.zeros_like(self.vec_master)
        self.vec_v = torch.zeros_like(self.vec_master)
        self.stage: Dict[str, torch.Tensor] = {}
        self.stage_flags: Dict[str, torch.Tensor] = {}
        self.stage_epoch: Dict[str, int] = {}
        for key in _STAGE_KEYS:
            name = key if key == "lm_head" else "layers.0." + key
            rows, cols = self.by_name[name].shape
            self.stage[key] = torch.empty((rows, cols), dtype=torch.bfloat16, device=self.device)
            self.stage_flags[key] = torch.zeros(4096, dtype=torch.int32, device=self.device)
            self.stage_epoch[key] = 0
        # ---- init: the same random stream as the single-GPU weights, each rank keeps its rows
        gen = torch.Generator(device=self.device).manual_seed(seed)
        for s in self.specs:
            n = math.prod(s.shape)
            if s.kind == "matrix":
                rows, cols = s.shape
                full = torch.empty(rows, cols, dtype=torch.float32, device=self.device).normal_(0.0, cfg.init_std, generator=gen)
                rpr = rows // W
                mine = full[self.rank * rpr:(self.rank + 1) * rpr].reshape(-1)
                so = self.shard_off[s.name]
                self.master[so:so + mine.numel()].copy_(mine)
                del full
            else:
                self.vec_master[s.offset:s.offset + n].fill_(1.0)
        self.sym_param.tensor.copy_(self.master)
        self.vec_p.copy_(self.vec_master)
        self.side = torch.cuda.Stream(device=self.device)
        self.flag_epoch = [0] * self.n_slots
        self.hyper = None
        self._pending = False
        self._trace, self._trace_done, self._trace_pos = [], False, 0
        self._progress = torch.zeros(4, dtype=torch.int32, device=self.device)
        self._progress_total = 0
        self.prefetch = os.environ.get("LT_FSDP_PREFETCH", "1") != "0"
        torch.cuda.synchronize()
        dist.barrier()

    # ------------------------------------------------------------------ views
    def _stage_key(self, name: str) -> str:
        return name if name == "lm_head" else name.split(".")[-1]

    def p(self, name: str) -> torch.Tensor:
        s = self.by_name[name]
        assert s.kind == "vector", "matrix parameters are sharded; use linear()/dgrad()"
        return self.vec_p[s.offset:s.offset + math.prod(s.shape)]

    def vector_grad(self, name: str) -> torch.Tensor:
        s = self.by_name[name]
        return self.vec_g[s.offset:s.offset + math.prod(s.shape)]

    def g(self, name: str) -> torch.Tensor:
        s = self.by_name[name]
        if s.kind == "vector":
            return self.vector_grad(name)
        o = self.full_off[name]
        return self.sym_grad.tensor[o:o + math.prod(s.shape)].view(*s.shape)

    def shard_view(self, flat: torch.Tensor, name: str) -> torch.Tensor:
        rows, cols = self.by_name[name].shape
        o = self.shard_off[name]
        return flat[o:o + (rows // self.world) * cols].view(rows // self.world, cols)

    # ------------------------------------------------------------------ GEMM providers
    def _gather_gemm(self, other, name, gather_operand, **kw):
        """One gather-GEMM.  The order of these calls is recorded during the first step; afterwards every call also
        tells its gather CTAs which operand the NEXT call needs, so that it is prefetched while this GEMM computes."""
        key = self._stage_key(name)
        rows, cols = self.by_name[name].shape
        self.stage_epoch[key] += 1
        M = other.shape[0]
        nxt = None
        if self._trace_done and not (self._trace_pos < len(self._trace) and self._trace[self._trace_pos] == (name, gather_operand)):
            # the call order changed (e.g. an evaluation pass): drop the schedule and void anything prefetched for it
            self._trace_done, self._trace, self._trace_pos = False, [], 0
            for k in self.stage_epoch:
                self.stage_epoch[k] += 2
        if self._trace_done:
            i = self._trace_pos
            if i + 1 < len(self._trace):
                n_name, n_op = self._trace[i + 1]
                n_key = self._stage_key(n_name)
                if n_key != key:
                    n_rows, n_cols = self.by_name[n_name].shape
                    nN, nK = (n_rows, n_cols) if n_op == 1 else (n_cols, n_rows)
                    nxt = K.make_next_gather(n_op, M, nN, nK, n_rows // self.world,
                                             self.sym_param.peer_ptrs(self.shard_off[n_name]), self.stage[n_key],
                                             self.stage_flags[n_key], self.stage_epoch[n_key] + 1)
            self._trace_pos += 1
        else:
            self._trace.append((name, gather_operand))
        N = rows if gather_operand == 1 else cols
        base = self._progress_total
        out = K.ag_gemm(None, self.stage[key], gather_operand=gather_operand,
                        shard_ptrs=self.sym_param.peer_ptrs(self.shard_off[name]), world=self.world, rank=self.rank,
                        rows_per_rank=rows // self.world, flags=self.stage_flags[key], epoch=self.stage_epoch[key],
                        other=other, n_comm=self.n_comm, next_gather=nxt, progress=self._progress, progress_base=base, **kw)
        self._progress_total = (base + 4 * K.gemm_num_tiles(M, N, self.n_comm)) & 0xFFFFFFFF
        return out

    def linear(self, x, name, **kw):
        return self._gather_gemm(x, name, 1, **kw)

    def dgrad(self, dy, name, **kw):
        return self._gather_gemm(dy, name, 2, **kw)

    def wgrad(self, dy, x, name, accumulate=False):
        return K.gemm(dy, x, a_major=1, b_major=1, out=self.g(name), accumulate=accumulate)

    def embedding(self, tokens):
        V, D = self.by_name["embed"].shape
        return K.embedding_fwd_sharded(tokens, self.sym_param.peer_ptrs(self.shard_off["embed"]), V, D, V // self.world,
                                       self.world)

    def zero_grad_embed(self):
        self.g("embed").zero_()

    def embedding_backward(self, tokens, dx):
        K.embedding_bwd(tokens, dx, self.g("embed"))

    # ------------------------------------------------------------------ fused reduce-scatter + AdamW
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
        if bucket == "head":
            return 1
        if bucket == "embed":
            return 2
        return 3 + int(bucket)

    def bucket_done(self, bucket):
        """All weight gradients of `bucket` have been issued on the current stream: reduce + update on the side stream."""
        if self.hyper is None:
            return
        h = self.hyper
        ev = torch.cuda.Event()
        ev.record()
        slot = self._slot(bucket)
        self.flag_epoch[slot] += 1
        segs = []
        for name in self._bucket_names(bucket):
            rows, cols = self.by_name[name].shape
            n = (rows // self.world) * cols
            segs.append((self.full_off[name] + self.rank * n, self.shard_off[name], n))
        with torch.cuda.stream(self.side):
            self.side.wait_event(ev)
            K.rs_adamw(self.sym_grad.ptrs, self.sym_grad.mc_ptr if self.use_multimem else None, self.master, self.m, self.v,
                       self.sym_param.tensor, segs, lr=h["lr"], beta1=h["beta1"], beta2=h["beta2"], eps=h["eps"],
                       wd=h["weight_decay"], step=h["step"], my_flags=self.sym_flags.tensor,
                       peer_flag_ptrs=self.sym_flags.ptrs, slot=slot, epoch=self.flag_epoch[slot], world=self.world,
                       rank=self.rank)
        self._pending = True

    def optimizer_step(self, *, lr, beta1, beta2, eps, weight_decay, step, dyn=None):
        if self.hyper is None:
            # gradients were accumulated without the fused path: reduce + update every bucket now
            self.begin_step(lr=lr, beta1=beta1, beta2=beta2, eps=eps, weight_decay=weight_decay, step=step)
            for b in ["head"] + list(reversed(range(self.cfg.n_layers))) + ["embed"]:
                self.bucket_done(b)
        dist.all_reduce(self.vec_g)
        K.adam_flat(self.vec_master, self.vec_g, self.vec_m, self.vec_v, self.vec_p, lr=lr, beta1=beta1, beta2=beta2, eps=eps,
                    wd=0.0, step=step, adamw=True, dyn=dyn)

    def finish_step(self):
        """Join the side stream and cross a node-wide barrier so that every shard is updated before the next gathers."""
        cur = torch.cuda.current_stream()
        if self._pending:
            cur.wait_stream(self.side)
            self._pending = False
        self.flag_epoch[self.SLOT_BARRIER] += 1
        K.signal_barrier(self.sym_flags.tensor, self.sym_flags.ptrs, self.SLOT_BARRIER, self.flag_epoch[self.SLOT_BARRIER],
                         self.world, self.rank)
        if self.hyper is not None and self.prefetch:
            self._trace_done = True          # one complete fused step has been seen: its call order is the schedule
        self._trace_pos = 0
        if not self._trace_done:
            self._trace = []
        self.hyper = None

    # ------------------------------------------------------------------ whole-model access (checkpoints, tests)
    def gather_full_master(self, name: str) -> torch.Tensor:
        s = self.by_name[name]
        if s.kind == "vector":
            return self.vec_master[s.offset:s.offset + math.prod(s.shape)].clone()
        mine = self.shard_view(self.master, name).contiguous()
        parts = [torch.empty_like(mine) for _ in range(self.world)]
        dist.all_gather(parts, mine)
        return torch.cat(parts, 0)

    def parameters(self) -> List[torch.Tensor]:
        return [self.gather_full_master(s.name) for s in self.specs]

    def load_parameters(self, tensors: List[torch.Tensor]) -> None:
        """Take whole parameters (in `specs` order, the same on every rank): each rank keeps its block of rows, as the
        initialisation does; then the bf16 shards are rebuilt (`after_load`)."""
        for s, t in zip(self.specs, tensors):
            n = math.prod(s.shape)
            if s.kind == "matrix":
                rows, cols = s.shape
                rpr = rows // self.world
                mine = t.view(rows, cols)[self.rank * rpr:(self.rank + 1) * rpr].to(self.device, torch.float32).reshape(-1)
                so = self.shard_off[s.name]
                self.master[so:so + mine.numel()].copy_(mine)
            else:
                self.vec_master[s.offset:s.offset + n].copy_(t.to(self.device, torch.float32).view(-1))
        self.after_load()

    def state_tensors(self) -> Dict[str, torch.Tensor]:
        """This rank's shard of the fp32 masters and AdamW moments plus the replicated vectors."""
        return {"master": self.master, "m": self.m, "v": self.v, "vec_master": self.vec_master, "vec_m": self.vec_m,
                "vec_v": self.vec_v}

    def after_load(self) -> None:
        """Rebuild the bf16 shards that the gathers read from the loaded masters; void anything staged or prefetched."""
        self.sym_param.tensor.copy_(self.master)
        self.vec_p.copy_(self.vec_master)
        for k in self.stage_epoch:
            self.stage_epoch[k] += 2
        torch.cuda.synchronize()
        dist.barrier()
