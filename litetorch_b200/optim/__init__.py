"""`lt.optim`: optimizers, LR schedulers and the optimizer-side GradScaler
(src/bindings/python_bindings.cpp:586-684, src/optim/*.cpp).

Parameters are `lt.Tensor`s.  fp32 CUDA parameters are updated by ONE native launch per step over a pointer
table (`lt_adam_table`) instead of one launch per tensor (src/optim/adamw.cpp:20-118 ->
optimizers.cu:49-78); bf16 parameters get fp32 master copies held by the optimizer.  CPU parameters use the
same update rule in PyTorch arithmetic.
"""
from __future__ import annotations

import math
from typing import List, Sequence

import torch

from ..amp import GradScaler as _AmpGradScaler
from ..core import Tensor, _unwrap


class Optimizer:
    def __init__(self, params: Sequence[Tensor], lr: float):
        self.params: List[Tensor] = list(params)
        self.lr = float(lr)
        self.step_count = 0

    def zero_grad(self):
        for p in self.params:
            p.zero_grad()

    def step(self):
        raise NotImplementedError

    def get_lr(self) -> float:
        return self.lr

    def set_lr(self, new_lr: float) -> None:
        self.lr = float(new_lr)

    def _tensors(self):
        return [_unwrap(p) for p in self.params]


def _flat_native(p) -> bool:
    """fp32 parameter and gradient, contiguous, on a CUDA device: the flat optimizer kernels apply."""
    g = p.grad
    return (p.is_cuda and p.dtype == torch.float32 and p.is_contiguous() and g is not None and g.dtype == torch.float32
            and g.is_contiguous())


class _QState:
    """Device-side bookkeeping of one tensor's quantised moments: two scale pairs (this step's and the next), the
    running absmax words and the e4m3 absmax history."""

    def __init__(self, p, code_dtype):
        dev = p.device
        self.mq = torch.zeros(p.shape, dtype=code_dtype, device=dev)
        self.vq = torch.zeros(p.shape, dtype=code_dtype, device=dev)
        self.scales = torch.ones(2, 2, dtype=torch.float32, device=dev)
        self.cur = 0
        self.amax = torch.zeros(2, dtype=torch.int32, device=dev)
        self.hist = torch.zeros(20, dtype=torch.float32, device=dev)
        self.hist_n = torch.zeros(1, dtype=torch.int32, device=dev)
        self.first = True


def _q_native(p) -> bool:
    g = p.grad
    return (p.is_cuda and p.is_contiguous() and p.dtype in (torch.float32, torch.bfloat16) and g is not None
            and g.is_contiguous() and g.dtype in (torch.float32, torch.bfloat16))


def _q_step(opt, i, p, fp8: bool):
    """One tensor's step on the GPU kernel; keeps `m_q / v_q / m_scale / v_scale` (or the e4m3 names) pointing at the
    live codes and device-resident scales so that checkpoints read them the usual way."""
    from ..ops import kernels as K
    st = opt._qstate[i]
    if st is None:
        st = opt._qstate[i] = _QState(p, torch.float8_e4m3fn if fp8 else torch.int8)
        codes_m, codes_v = (opt.m8, opt.v8) if fp8 else (opt.m_q, opt.v_q)
        if codes_m[i] is not None:                       # state loaded from a checkpoint or left by the torch path
            st.mq.copy_(codes_m[i])
            st.vq.copy_(codes_v[i])
            st.scales[0, 0], st.scales[0, 1] = float(opt.m_scale[i]), float(opt.v_scale[i])
            st.first = False
            if fp8:
                for k, h in enumerate((opt.m_hist[i], opt.v_hist[i])):
                    for j, a in enumerate(h[-10:]):
                        st.hist[k * 10 + j] = a
                st.hist_n.fill_(min(len(opt.m_hist[i]), 10))
    old, new = st.scales[st.cur], st.scales[1 - st.cur]
    K.adam_q8(p, p.grad, st.mq, st.vq, lr=opt.lr, beta1=opt.beta1, beta2=opt.beta2, eps=opt.eps, wd=opt.weight_decay,
              step=opt.step_count, fp8=fp8, first=st.first, scale_old=old, scale_new=new, amax=st.amax, hist=st.hist,
              hist_n=st.hist_n)
    st.cur, st.first = 1 - st.cur, False
    if fp8:
        opt.m8[i], opt.v8[i] = st.mq, st.vq
    else:
        opt.m_q[i], opt.v_q[i] = st.mq, st.vq
    opt.m_scale[i], opt.v_scale[i] = new[0], new[1]      # 0-dim device tensors: no host sync


class SGD(Optimizer):
    def __init__(self, params, lr: float = 0.01, momentum: float = 0.0, weight_decay: float = 0.0):
        super().__init__(params, lr)
        self.momentum, self.weight_decay = momentum, weight_decay
        self.velocity = [None] * len(self.params)

    @torch.no_grad()
    def step(self):
        self.step_count += 1
        for i, p in enumerate(self._tensors()):
            if p.grad is None:
                continue
            if _flat_native(p):
                # one fused pass on the GPU (sgd_step_kernel of the reference: src/backend/gpu_native/optim/optimizers.cu:87-104)
                from ..ops import kernels as K
                if self.momentum and self.velocity[i] is None:
                    self.velocity[i] = torch.zeros_like(p)
                K.sgd_flat(p, p.grad, self.velocity[i] if self.momentum else None, lr=self.lr, momentum=self.momentum,
                           wd=self.weight_decay)
                continue
            g = p.grad.to(p.dtype)
            if self.weight_decay:
                g = g + self.weight_decay * p
            if self.momentum:
                if self.velocity[i] is None:
                    self.velocity[i] = torch.zeros_like(p)
                self.velocity[i].mul_(self.momentum).add_(g)
                g = self.velocity[i]
            p.add_(g, alpha=-self.lr)


class _AdamBase(Optimizer):
    decoupled = False

    def __init__(self, params, lr=0.001, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0):
        super().__init__(params, lr)
        self.beta1, self.beta2, self.eps, self.weight_decay = beta1, beta2, eps, weight_decay
        self.m = [None] * len(self.params)
        self.v = [None] * len(self.params)
        self.master = [None] * len(self.params)  # fp32 master copies of low-precision parameters
        self._pver = [None] * len(self.params)   # version counter of each low-precision parameter after our last write
        self._table = None

    def _state_device(self, p):
        return p.device

    def _ensure_state(self, i, p):
        if self.m[i] is None:
            dev = self._state_device(p)
            self.m[i] = torch.zeros(p.shape, dtype=torch.float32, device=dev)
            self.v[i] = torch.zeros(p.shape, dtype=torch.float32, device=dev)
            if p.dtype != torch.float32:
                self.master[i] = p.detach().to(device=dev, dtype=torch.float32).clone()
                self._pver[i] = p._version

    def _refresh_masters(self, ts):
        """A low-precision parameter that was written by someone else since our last step (a checkpoint load, a manual
        copy_) no longer matches its fp32 master: take over the new values.  Elements whose master still rounds to the
        parameter keep their extra fp32 bits, so loading the same checkpoint into both is exact in either order."""
        for i, p in enumerate(ts):
            mst = self.master[i]
            if mst is None or self._pver[i] == p._version:
                continue
            cur = p.detach().to(mst.device)
            stale = mst.to(p.dtype) != cur
            if bool(stale.any()):
                mst[stale] = cur[stale].float()
            self._pver[i] = p._version

    def _mark_versions(self, ts):
        for i, p in enumerate(ts):
            if self.master[i] is not None:
                self._pver[i] = p._version

    def _native_ok(self, ts):
        for t in ts:
            if not (t.is_cuda and t.is_contiguous() and t.dtype in (torch.float32, torch.bfloat16)):
                return False
            if t.grad is not None and not (t.grad.is_contiguous() and t.grad.dtype in (torch.float32, torch.bfloat16)):
                return False
            if self._state_device(t) != t.device:
                return False
        return True

    def _step_native(self, ts):
        from ..ops import kernels as K
        live = [i for i, t in enumerate(ts) if t.grad is not None]
        if not live:
            return
        for i in live:
            self._ensure_state(i, ts[i])
        # The table is keyed on the parameters only: gradients are usually freed every step (`zero_grad` drops them) and
        # come back at other addresses, and rebuilding the per-chunk arrays for that would cost more than the update.
        key = tuple((ts[i].data_ptr(), ts[i].grad.dtype) for i in live)
        gptrs = tuple(ts[i].grad.data_ptr() for i in live)
        if self._table is not None and self._table[0] == key and self._table[1]["gptrs"] != gptrs:
            tab = self._table[1]
            tab["g"] = torch.tensor(gptrs, dtype=torch.int64, device=tab["g"].device)
            tab["gptrs"] = gptrs
        if self._table is None or self._table[0] != key:
            dev = ts[live[0]].device
            chunk = K._fn("lt_adam_chunk_elems")()
            P = [(self.master[i] if self.master[i] is not None else ts[i]) for i in live]
            i64 = lambda v: torch.tensor(v, dtype=torch.int64, device=dev)  # noqa: E731
            tab = {"p": i64([t.data_ptr() for t in P]), "g": i64([ts[i].grad.data_ptr() for i in live]),
                   "m": i64([self.m[i].data_ptr() for i in live]), "v": i64([self.v[i].data_ptr() for i in live]),
                   "p16": i64([ts[i].data_ptr() if self.master[i] is not None else 0 for i in live]),
                   "numel": i64([ts[i].numel() for i in live]),
                   "gbf": torch.tensor([1 if ts[i].grad.dtype == torch.bfloat16 else 0 for i in live], dtype=torch.int32, device=dev),
                   "has16": any(self.master[i] is not None for i in live), "gptrs": gptrs}
            ct, co = [], []
            for k, i in enumerate(live):
                for off in range(0, ts[i].numel(), chunk):
                    ct.append(k)
                    co.append(off)
            tab["ct"] = torch.tensor(ct, dtype=torch.int32, device=dev)
            tab["co"] = i64(co)
            self._table = (key, tab)
        tab = self._table[1]
        rc = K._fn("lt_adam_table")(tab["p"].data_ptr(), tab["g"].data_ptr(), tab["m"].data_ptr(), tab["v"].data_ptr(),
                                    tab["p16"].data_ptr() if tab["has16"] else None, tab["numel"].data_ptr(),
                                    tab["gbf"].data_ptr(), tab["ct"].data_ptr(), tab["co"].data_ptr(), tab["ct"].numel(),
                                    self.lr, self.beta1, self.beta2, self.eps, self.weight_decay,
                                    1.0 - self.beta1 ** self.step_count, 1.0 - self.beta2 ** self.step_count,
                                    1 if self.decoupled else 0, None, torch.cuda.current_stream().cuda_stream)
        K._check(rc, "lt_adam_table")

    def _step_torch(self, ts, offset: int = 0):
        bc1 = 1.0 - self.beta1 ** self.step_count
        bc2 = 1.0 - self.beta2 ** self.step_count
        for i, p in enumerate(ts, start=offset):
            if p.grad is None:
                continue
            self._ensure_state(i, p)
            dev = self.m[i].device
            if self.master[i] is not None:
                w = self.master[i]
            elif p.device == dev:
                w = p
            else:
                w = p.detach().to(dev, torch.float32)
            g = p.grad.detach().to(dev, torch.float32)
            if not self.decoupled and self.weight_decay:
                g = g + self.weight_decay * w
            self.m[i].mul_(self.beta1).add_(g, alpha=1 - self.beta1)
            self.v[i].mul_(self.beta2).addcmul_(g, g, value=1 - self.beta2)
            if self.decoupled and self.weight_decay:
                w.mul_(1 - self.lr * self.weight_decay)
            w.addcdiv_(self.m[i] / bc1, (self.v[i] / bc2).sqrt_().add_(self.eps), value=-self.lr)
            if w is not p:
                p.copy_(w.to(p.device, p.dtype))

    @torch.no_grad()
    def step(self):
        self.step_count += 1
        ts = self._tensors()
        self._refresh_masters(ts)
        if ts and self._native_ok(ts):
            self._step_native(ts)
        else:
            self._step_torch(ts)
        self._mark_versions(ts)


class Adam(_AdamBase):
    decoupled = False


class AdamW(_AdamBase):
    """Decoupled weight decay, bias-corrected.  `offload_to_cpu` keeps m, v (and masters) in host memory."""
    decoupled = True

    def __init__(self, params, lr=0.001, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01, offload_to_cpu=False,
                 state_limit_bytes: int = 0):
        """state_limit_bytes > 0: the moments live under an `lt.memory.ResidencyManager` with that device-memory limit -
        at most that many bytes of m / v are on the device at a time, the least recently used tensors wait in pinned
        host memory and are swapped in for their parameter's update (the reference's storage eviction,
        src/memory_manager/memory_manager.cpp:54-107, applied to optimizer state)."""
        super().__init__(params, lr, beta1, beta2, eps, weight_decay)
        self.offload_to_cpu = offload_to_cpu
        self._mm = None
        self._handles = {}
        if state_limit_bytes > 0:
            from ..memory import ResidencyManager
            dev = next((t.device for t in self._tensors()), torch.device("cpu"))
            self._mm = ResidencyManager(state_limit_bytes, dev)

    @torch.no_grad()
    def step(self):
        if self._mm is None:
            return super().step()
        self.step_count += 1
        ts = self._tensors()
        self._refresh_masters(ts)
        for i, p in enumerate(ts):
            if p.grad is None:
                continue
            if i not in self._handles:
                self._ensure_state(i, p)
                self._handles[i] = (self._mm.register(self.m[i]), self._mm.register(self.v[i]))
                self.m[i] = self.v[i] = None          # the manager's handles are now the only owners
            hm, hv = self._handles[i]
            with self._mm.use(hm) as m, self._mm.use(hv) as v:
                self.m[i], self.v[i] = m, v
                self._step_torch([p], offset=i)
                self.m[i] = self.v[i] = None
        self._mark_versions(ts)

    def _state_device(self, p):
        return torch.device("cpu") if self.offload_to_cpu else p.device


class RMSprop(Optimizer):
    def __init__(self, params, lr=0.01, alpha=0.99, eps=1e-8, weight_decay=0.0):
        super().__init__(params, lr)
        self.alpha, self.eps, self.weight_decay = alpha, eps, weight_decay
        self.square_avg = [None] * len(self.params)

    @torch.no_grad()
    def step(self):
        self.step_count += 1
        for i, p in enumerate(self._tensors()):
            if p.grad is None:
                continue
            if self.square_avg[i] is None:
                self.square_avg[i] = torch.zeros_like(p, dtype=torch.float32)
            if _flat_native(p):
                # rmsprop_step_kernel of the reference (src/backend/gpu_native/optim/optimizers.cu:106-124), one pass
                from ..ops import kernels as K
                K.rmsprop_flat(p, p.grad, self.square_avg[i], lr=self.lr, alpha=self.alpha, eps=self.eps, wd=self.weight_decay)
                continue
            g = p.grad.float()
            if self.weight_decay:
                g = g + self.weight_decay * p.float()
            self.square_avg[i].mul_(self.alpha).addcmul_(g, g, value=1 - self.alpha)
            p.add_((g / (self.square_avg[i].sqrt() + self.eps)).to(p.dtype), alpha=-self.lr)


class AdamW8bit(_AdamBase):
    """AdamW whose m and v are stored as int8 codes with one absmax scale per tensor (75 % less state memory);
    the update itself runs in fp32 (src/optim/adamw_8bit.cpp:13-104)."""
    decoupled = True

    def __init__(self, params, lr=0.001, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0):
        super().__init__(params, lr, beta1, beta2, eps, weight_decay)
        n = len(self.params)
        self.m_q, self.v_q = [None] * n, [None] * n
        self.m_scale, self.v_scale = [1.0] * n, [1.0] * n
        self._qstate = [None] * n

    @staticmethod
    def _quant(x):
        amax = float(x.abs().max())
        scale = amax / 127.0 if amax > 0 else 1.0
        return torch.clamp(torch.round(x / scale), -127, 127).to(torch.int8), scale

    @torch.no_grad()
    def step(self):
        self.step_count += 1
        bc1, bc2 = 1 - self.beta1 ** self.step_count, 1 - self.beta2 ** self.step_count
        for i, p in enumerate(self._tensors()):
            if p.grad is None:
                continue
            if _q_native(p):
                _q_step(self, i, p, fp8=False)
                continue
            g = p.grad.float()
            m = self.m_q[i].float() * self.m_scale[i] if self.m_q[i] is not None else torch.zeros_like(g)
            v = self.v_q[i].float() * self.v_scale[i] if self.v_q[i] is not None else torch.zeros_like(g)
            m.mul_(self.beta1).add_(g, alpha=1 - self.beta1)
            v.mul_(self.beta2).addcmul_(g, g, value=1 - self.beta2)
            w = p.float()
            w.mul_(1 - self.lr * self.weight_decay)
            w.addcdiv_(m / bc1, (v / bc2).sqrt() + self.eps, value=-self.lr)
            p.copy_(w.to(p.dtype))
            self.m_q[i], self.m_scale[i] = self._quant(m)
            self.v_q[i], self.v_scale[i] = self._quant(v)

    def state_bytes(self) -> int:
        return sum(q.numel() for q in self.m_q if q is not None) + sum(q.numel() for q in self.v_q if q is not None)


class AdamWFP8(_AdamBase):
    """AdamW with e4m3 moment storage and delayed scaling from a 10-step amax history (scale = amax / 240)
    (src/optim/adamw_fp8.cpp:13-126)."""
    decoupled = True
    HISTORY = 10

    def __init__(self, params, lr=0.001, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0):
        self.m8, self.v8 = [], []
        super().__init__(params, lr, beta1, beta2, eps, weight_decay)
        n = len(self.params)
        self.m8, self.v8 = [None] * n, [None] * n
        self.m_scale, self.v_scale = [1.0] * n, [1.0] * n
        self.m_hist, self.v_hist = [[] for _ in range(n)], [[] for _ in range(n)]
        self._qstate = [None] * n

    # `m` / `v` read as the e4m3 moment tensors, as the reference's public members do (include/litetorch/optim.h)
    @property
    def m(self):
        return [None if t is None else Tensor(t) for t in self.m8]

    @m.setter
    def m(self, _):
        pass

    @property
    def v(self):
        return [None if t is None else Tensor(t) for t in self.v8]

    @v.setter
    def v(self, _):
        pass

    def _store(self, x, hist):
        hist.append(float(x.abs().max()))
        del hist[:-self.HISTORY]
        amax = max(hist)
        scale = amax / 240.0 if amax > 0 else 1.0
        return (x / scale).clamp(-448, 448).to(torch.float8_e4m3fn), scale

    @torch.no_grad()
    def step(self):
        self.step_count += 1
        bc1, bc2 = 1 - self.beta1 ** self.step_count, 1 - self.beta2 ** self.step_count
        for i, p in enumerate(self._tensors()):
            if p.grad is None:
                continue
            if _q_native(p):
                _q_step(self, i, p, fp8=True)
                continue
            g = p.grad.float()
            m = self.m8[i].float() * self.m_scale[i] if self.m8[i] is not None else torch.zeros_like(g)
            v = self.v8[i].float() * self.v_scale[i] if self.v8[i] is not None else torch.zeros_like(g)
            m.mul_(self.beta1).add_(g, alpha=1 - self.beta1)
            v.mul_(self.beta2).addcmul_(g, g, value=1 - self.beta2)
            w = p.float()
            w.mul_(1 - self.lr * self.weight_decay)
            w.addcdiv_(m / bc1, (v / bc2).sqrt() + self.eps, value=-self.lr)
            p.copy_(w.to(p.dtype))
            self.m8[i], self.m_scale[i] = self._store(m, self.m_hist[i])
            self.v8[i], self.v_scale[i] = self._store(v, self.v_hist[i])


class ZeRO3Optimizer(_AdamBase):
    """Adam over sharded parameters: tensors that carry a `.shard` (set by FullyShardedDataParallel) update the shard
    with the shard's gradient; replicated tensors are updated by the owner rank `index % world` and broadcast
    (src/optim/zero3_optimizer.cpp:11-105)."""
    decoupled = True

    @torch.no_grad()
    def step(self):
        import torch.distributed as dist
        self.step_count += 1
        world = dist.get_world_size() if dist.is_initialized() else 1
        rank = dist.get_rank() if dist.is_initialized() else 0
        bc1, bc2 = 1 - self.beta1 ** self.step_count, 1 - self.beta2 ** self.step_count
        for i, lp in enumerate(self.params):
            shard = getattr(lp, "shard", None)
            tgt = _unwrap(shard) if shard is not None else _unwrap(lp)
            g = tgt.grad
            owner = i % world
            if shard is None and world > 1:
                if rank == owner and g is not None:
                    self._one(i, tgt, g, bc1, bc2)
                dist.broadcast(tgt, src=owner)
            elif g is not None:
                self._one(i, tgt, g, bc1, bc2)

    def _one(self, i, p, g, bc1, bc2):
        self._ensure_state(i, p)
        g = g.float()
        self.m[i].mul_(self.beta1).add_(g, alpha=1 - self.beta1)
        self.v[i].mul_(self.beta2).addcmul_(g, g, value=1 - self.beta2)
        w = p.float()
        w.mul_(1 - self.lr * self.weight_decay)
        w.addcdiv_(self.m[i] / bc1, (self.v[i] / bc2).sqrt() + self.eps, value=-self.lr)
        p.copy_(w.to(p.dtype))


class StepLR:
    def __init__(self, optimizer: Optimizer, step_size: int, gamma: float = 0.1):
        self.optimizer, self.step_size, self.gamma = optimizer, step_size, gamma
        self.base_lr, self.last_epoch = optimizer.lr, 0      # `last_epoch`: steps taken, the reference's field (include/litetorch/optim.h:131)

    @property
    def epoch(self) -> int:
        return self.last_epoch

    def step(self):
        self.last_epoch += 1
        self.optimizer.lr = self.base_lr * (self.gamma ** (self.last_epoch // self.step_size))

    def get_lr(self) -> float:
        return self.optimizer.lr


class CosineAnnealingLR:
    def __init__(self, optimizer: Optimizer, T_max: int, eta_min: float = 0.0):
        self.optimizer, self.T_max, self.eta_min = optimizer, T_max, eta_min
        self.base_lr, self.last_epoch = optimizer.lr, 0

    @property
    def epoch(self) -> int:
        return self.last_epoch

    def step(self):
        self.last_epoch += 1
        t = min(self.last_epoch, self.T_max)
        self.optimizer.lr = self.eta_min + (self.base_lr - self.eta_min) * (1 + math.cos(math.pi * t / self.T_max)) / 2

    def get_lr(self) -> float:
        return self.optimizer.lr


class WarmupCosineLR:
    """Linear warm-up from 0 to the optimizer's rate over `warmup_steps`, then half a cosine down to `min_lr_ratio` times
    that rate at `total_steps` (constant afterwards): the usual schedule of LLM pre-training.  The rate is a function of
    `last_epoch` alone, so a resumed job sets `last_epoch` to its step count and continues on the same curve.  Unlike the
    two schedulers of the reference it also sets the rate of step 0 at construction (a warm-up starts below the base rate)."""

    def __init__(self, optimizer, warmup_steps: int, total_steps: int, min_lr_ratio: float = 0.1, last_epoch: int = 0):
        self.optimizer, self.warmup_steps, self.total_steps = optimizer, int(warmup_steps), int(total_steps)
        self.min_lr_ratio, self.base_lr = float(min_lr_ratio), optimizer.lr
        self.last_epoch = int(last_epoch)
        self.optimizer.lr = self.lr_at(self.last_epoch)

    def lr_at(self, step: int) -> float:
        if step < self.warmup_steps:
            return self.base_lr * (step + 1) / self.warmup_steps
        t = (step - self.warmup_steps) / max(1, self.total_steps - self.warmup_steps)
        return self.base_lr * (self.min_lr_ratio + (1.0 - self.min_lr_ratio) * 0.5 * (1.0 + math.cos(math.pi * min(t, 1.0))))

    @property
    def epoch(self) -> int:
        return self.last_epoch

    def step(self):
        self.last_epoch += 1
        self.optimizer.lr = self.lr_at(self.last_epoch)

    def get_lr(self) -> float:
        return self.optimizer.lr


class GradScaler(_AmpGradScaler):
    """`lt.optim.GradScaler`: `scale_loss / step / update` and the `.scale` value (src/optim/grad_scaler.cpp:8-79)."""

    def scale_loss(self, loss: Tensor) -> Tensor:
        return Tensor(_unwrap(loss) * self._scale)

    scale = property(lambda self: self._scale, lambda self, v: setattr(self, "_scale", float(v)))


__all__ = ["Optimizer", "SGD", "Adam", "AdamW", "AdamW8bit", "AdamWFP8", "RMSprop", "ZeRO3Optimizer", "StepLR",
           "CosineAnnealingLR", "WarmupCosineLR", "GradScaler"]
