"""`Trainer`: the public training entry point (host batches in, loss out).

    tr = Trainer(LlamaConfig.llama_1b())          # one process per GPU; reads RANK/LOCAL_RANK/WORLD_SIZE
    loss = tr.step(tokens_cpu, targets_cpu)       # pinned host int64 [B, T] -> float

`step` copies the batch from pinned host memory, runs forward + backward + AdamW on the sm_100a kernels
(ZeRO-3 sharded over the process group when world_size > 1; with `tp > 1` the ranks form a dp x tp mesh, matrices are
cut over the tp axis with sequence parallelism and their slices are ZeRO-3 sharded over the dp axis) and reads the
loss back.  Every rank of a tensor-parallel group must be given the same batch.
The reference's equivalent is the hand-written loop `zero_grad / forward / backward / step / loss.item()`
of its example trainers (train_cat_dog.py:312-319).
"""
from __future__ import annotations

import os
import time
from typing import Optional

import torch

from .models.llama import LlamaConfig, LlamaEngine


def _local_weights():
    from .models.llama import LocalWeights
    return LocalWeights


class Trainer:
    def __init__(self, cfg: LlamaConfig, *, lr: float = 3e-4, betas=(0.9, 0.95), eps: float = 1e-8,
                 weight_decay: float = 0.1, seed: int = 0, activation_checkpointing: bool = False,
                 device: Optional[str] = None, parallel: str = "auto", tp: int = 1, param_dtype=torch.bfloat16,
                 micro_batches: int = 1, grad_clip: float = 0.0):
        self.micro_batches = max(1, int(micro_batches))     # default split of a `step` batch (gradient accumulation)
        self.rank = int(os.environ.get("RANK", "0"))
        self.world_size = int(os.environ.get("WORLD_SIZE", "1"))
        local = int(os.environ.get("LOCAL_RANK", "0"))
        self.device = torch.device(device) if device else torch.device("cuda", local)
        if self.device.type == "cuda":
            torch.cuda.set_device(self.device)
        self.cfg = cfg
        weights = None
        self.tp = tp
        self.dp = 1
        if self.world_size > 1 and parallel in ("auto", "fsdp", "hybrid"):
            import torch.distributed as dist
            from .parallel.fsdp import ShardedWeights, ensure_process_group
            if not dist.is_initialized() and self.device.type != "cuda":
                dist.init_process_group("gloo")
            ensure_process_group()
            if tp > 1 or parallel == "hybrid" or self.device.type != "cuda":
                from .parallel.hybrid import HybridWeights
                weights = HybridWeights(cfg, self.device, tp=tp, seed=seed, param_dtype=param_dtype)
            else:
                weights = ShardedWeights(cfg, self.device, seed=seed)
            self.dp = self.world_size // tp
        self.dp_rank = self.rank // tp
        if weights is None and (param_dtype != torch.bfloat16 or self.device.type != "cuda"):
            from .models.llama import LocalWeights
            weights = LocalWeights(cfg, self.device, seed, param_dtype=param_dtype)
        self.engine = LlamaEngine(cfg, self.device, weights=weights, seed=seed, lr=lr, betas=betas, eps=eps,
                                  weight_decay=weight_decay, activation_checkpointing=activation_checkpointing,
                                  world_size=self.dp, grad_clip=grad_clip)
        self._tok = None
        self._tgt = None
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        self._metrics, self._step_no, self._last_t = None, 0, None

    @classmethod
    def from_config(cls, run, **kw) -> "Trainer":
        """Build the trainer of a `config.RunConfig` (a preset name or JSON path is loaded first).  This entry point
        covers the dp (ZeRO-3) x tp (+ sequence parallel) layouts of the hand-scheduled Llama engine; layouts with
        context, expert or pipeline parallelism run through `models/run_config.py`."""
        from . import config as _config
        if isinstance(run, str):
            run = _config.load(run)
        p = run.parallel
        if p.pp * p.cp * max(p.ep, 1) != 1:
            raise ValueError("Trainer.from_config runs dp (ZeRO-3) x tp layouts; use models.run_config for pp/cp/ep")
        o = run.optim
        return cls(run.llama_config(), lr=o.lr, betas=(o.beta1, o.beta2), eps=o.eps, weight_decay=o.weight_decay,
                   seed=run.seed, activation_checkpointing=run.activation_checkpointing,
                   parallel=("hybrid" if p.tp > 1 else "fsdp") if (p.zero_stage >= 1 or p.tp > 1) else "none", tp=p.tp,
                   **dict({"micro_batches": getattr(run, "micro_batches", 1), "grad_clip": o.grad_clip}, **kw))

    # The learning rate lives in the engine and is read at every optimizer step; with these three members a trainer can
    # stand where the LR schedulers expect an optimizer: `lt.optim.CosineAnnealingLR(trainer, T_max=...)`.
    @property
    def lr(self) -> float:
        return self.engine.lr

    @lr.setter
    def lr(self, value: float) -> None:
        self.engine.lr = float(value)

    def get_lr(self) -> float:
        return self.engine.lr

    def set_lr(self, new_lr: float) -> None:
        self.engine.lr = float(new_lr)

    def step_device(self, tokens: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        """Batch already on the device; returns the loss as a device scalar (no host sync)."""
        return self.engine.train_step(tokens, targets)

    def step(self, tokens_cpu: torch.Tensor, targets_cpu: torch.Tensor, micro_batches: Optional[int] = None) -> float:
        """One optimizer step on a host batch: copy in, train, read the loss back.  micro_batches > 1 splits the batch along
        its first axis and accumulates the gradients (`LlamaEngine.train_step_accumulated`; checked against the one-batch step
        on CPU and gloo ranks)."""
        if self._tok is None or self._tok.shape != tokens_cpu.shape:
            self._tok = torch.empty(tokens_cpu.shape, dtype=torch.int64, device=self.device)
            self._tgt = torch.empty(targets_cpu.shape, dtype=torch.int64, device=self.device)
        self._tok.copy_(tokens_cpu, non_blocking=True)
        self._tgt.copy_(targets_cpu, non_blocking=True)
        self.h2d_bytes = tokens_cpu.numel() * tokens_cpu.element_size() + targets_cpu.numel() * targets_cpu.element_size()
        micro_batches = self.micro_batches if micro_batches is None else int(micro_batches)
        if micro_batches > 1:
            if tokens_cpu.shape[0] % micro_batches:
                raise ValueError("%d sequences do not split into %d micro-batches" % (tokens_cpu.shape[0], micro_batches))
            loss = self.engine.train_step_accumulated(list(zip(self._tok.chunk(micro_batches), self._tgt.chunk(micro_batches))))
        else:
            loss = self.engine.train_step(self._tok, self._tgt)
        out = loss.float().cpu()
        self.d2h_bytes = out.numel() * out.element_size()
        if self._metrics is not None:
            now = time.perf_counter()
            self._step_no += 1
            rec = {"step": self._step_no, "loss": float(out)}
            if self._last_t is not None:          # host time between two loss read-backs = one full step
                ms = (now - self._last_t) * 1e3
                rec.update(step_ms=round(ms, 3), tokens_per_s=round(tokens_cpu.numel() * self.dp / ms * 1e3, 1))
            self._last_t = now
            self._metrics.write(**rec)
        return float(out)

    def evaluate(self, tokens_cpu: torch.Tensor, targets_cpu: torch.Tensor, reduce: bool = True) -> float:
        """Loss of a host batch without an update (`LlamaEngine.eval_loss`).  Under data parallelism every replica
        evaluates its own batch; `reduce` (default) averages the result over all ranks (the ranks of a tensor-parallel
        group hold the same value, so this is the mean over the replicas) - every rank must then call it."""
        dev = self.device
        out = self.engine.eval_loss(tokens_cpu.to(dev, non_blocking=True), targets_cpu.to(dev, non_blocking=True))
        if reduce and self.world_size > 1 and not isinstance(self.engine.w, _local_weights()):
            import torch.distributed as dist
            out = out.detach().clone().reshape(1)
            dist.all_reduce(out)
            out = out / self.world_size
        return float(out)

    # ---- checkpoint / resume of the whole training state
    def _layout(self) -> dict:
        from dataclasses import asdict
        return {"weights": type(self.engine.w).__name__, "world_size": self.world_size if self.engine.w.__class__.__name__ != "LocalWeights" else 1,
                "tp": self.tp, "model": asdict(self.cfg)}

    def save(self, directory: str, keep: int = 2, loader=None, background: bool = False) -> None:
        """Write everything a restart needs: per rank, its fp32 master weights and AdamW moments (the shard it owns
        under ZeRO-3 / tensor parallelism, the replicated norm gains included) as one LTW1 file, and by rank 0 a
        manifest with the model, the layout and the optimizer's step count (bias correction depends on it).

        A checkpoint is a sub-directory `step-<n>`: every rank writes into `.step-<n>.tmp`, and once all files are on disk
        rank 0 renames it and points the file `LATEST` at it (both atomic), then drops all but the newest `keep`
        checkpoints.  A job that dies in the middle of a save therefore leaves the previous checkpoint intact and
        `load` never sees a mix of two steps.  `loader`: an `lt.data.DataLoader` whose position (epoch, permutation, next
        index: the LTDL record) is stored per rank next to the tensors and restored by `load(..., loader=...)`.

        `background=True`: the state is copied to host memory now (the checkpoint is of THIS step), the file is written by
        a thread while training goes on, and the checkpoint is published (barrier of the ranks, renames) by
        `finish_save()` - called explicitly, or by the next `save` / `load`.  Until then `LATEST` names the previous one."""
        import shutil
        from .serialization import save_sharded
        self.finish_save()
        w = self.engine.w
        state = w.state_tensors()
        lay = self._layout()
        sharded = lay["world_size"] > 1
        if self.device.type == "cuda":
            torch.cuda.synchronize()
        name = "step-%08d" % self.engine.step_count
        tmp, final = os.path.join(directory, "." + name + ".tmp"), os.path.join(directory, name)
        meta = dict(lay, names=list(state), step_count=self.engine.step_count)
        rank = self.rank if sharded else 0
        # private host copies: a CPU fp32 tensor would otherwise be written while later steps change it
        snapshot = [t.detach().to("cpu", torch.float32, copy=True) for t in state.values()]
        os.makedirs(tmp, exist_ok=True)
        if loader is not None:
            loader.save_state(os.path.join(tmp, "loader.rank%05d.ltdl" % rank))

        def write():
            save_sharded(tmp, snapshot, rank, lay["world_size"], tag="trainer", meta=meta)

        def publish():
            if sharded:
                import torch.distributed as dist
                dist.barrier()                                   # every rank's file is in the temporary directory
            if not sharded or self.rank == 0:
                if os.path.isdir(final):
                    shutil.rmtree(final)                         # the same step saved twice
                os.replace(tmp, final)
                with open(os.path.join(directory, "LATEST.tmp"), "w") as f:
                    f.write(name)
                os.replace(os.path.join(directory, "LATEST.tmp"), os.path.join(directory, "LATEST"))
                done = sorted(d for d in os.listdir(directory) if d.startswith("step-") and os.path.isdir(os.path.join(directory, d)))
                for d in done[:-keep] if keep > 0 else []:
                    if d != name:
                        shutil.rmtree(os.path.join(directory, d), ignore_errors=True)
                for d in os.listdir(directory):                  # leftovers of saves that never finished
                    if d.startswith(".step-") and d.endswith(".tmp") and d != "." + name + ".tmp":
                        shutil.rmtree(os.path.join(directory, d), ignore_errors=True)
            if sharded:
                import torch.distributed as dist
                dist.barrier()

        if not background:
            write()
            publish()
            return
        import threading
        box = {}

        def run():
            try:
                write()
            except BaseException as e:                           # re-raised on the training thread by finish_save
                box["error"] = e
        th = threading.Thread(target=run, name="lt-checkpoint-writer", daemon=False)
        th.start()
        self._pending_save = (th, box, publish)

    def finish_save(self) -> None:
        """Wait for a `save(..., background=True)` that is still writing and publish its checkpoint (all ranks call this at
        the same step: it contains the barrier).  Raises what the writer thread raised.  A no-op otherwise."""
        pending, self._pending_save = getattr(self, "_pending_save", None), None
        if pending is None:
            return
        th, box, publish = pending
        th.join()
        if "error" in box:
            raise box["error"]
        publish()

    @staticmethod
    def latest_checkpoint(directory: str):
        """The sub-directory `LATEST` points at, `directory` itself for a flat checkpoint, None when there is none."""
        try:
            with open(os.path.join(directory, "LATEST")) as f:
                d = os.path.join(directory, f.read().strip())
            return d if os.path.isdir(d) else None
        except OSError:
            return directory if os.path.exists(os.path.join(directory, "trainer.manifest.json")) else None

    def load(self, directory: str, loader=None) -> None:
        """Resume from `save`: the checkpoint must come from the same model on the same layout (world size, tp)."""
        import json
        from .serialization import CheckpointError, load_sharded
        self.finish_save()
        w = self.engine.w
        state = w.state_tensors()
        lay = self._layout()
        root = directory
        directory = self.latest_checkpoint(root)
        if directory is None:
            raise CheckpointError("no finished checkpoint in %s" % root)
        with open(os.path.join(directory, "trainer.manifest.json")) as f:
            meta = json.load(f)["meta"]
        for k in ("weights", "world_size", "tp", "model"):
            if meta.get(k) != lay[k]:
                raise CheckpointError("checkpoint %s differs: written with %r, this trainer has %r (another world size or "
                                      "tensor-parallel width: `python -m litetorch_b200.checkpoint_tools reshard`)"
                                      % (k, meta.get(k), lay[k]))
        if meta["names"] != list(state):
            raise CheckpointError("checkpoint holds %r, this trainer expects %r" % (meta["names"], list(state)))
        sharded = lay["world_size"] > 1
        tensors = load_sharded(directory, self.rank if sharded else 0, lay["world_size"], tag="trainer")
        for (name, dst), src in zip(state.items(), tensors):
            if src.numel() != dst.numel():
                raise CheckpointError("%s: %d elements in the file, %d in this trainer" % (name, src.numel(), dst.numel()))
            dst.copy_(src.view_as(dst))
        self.engine.step_count = int(meta["step_count"])
        w.after_load()
        if loader is not None:
            path = os.path.join(directory, "loader.rank%05d.ltdl" % (self.rank if sharded else 0))
            if not os.path.exists(path):
                raise CheckpointError("the checkpoint holds no data-loader state for rank %d" % self.rank)
            loader.load_state(path)

    def log_metrics(self, path: str) -> None:
        """Append one JSON line per `step` (step, loss, step_ms, tokens_per_s, allocator high-water mark) to `path`."""
        from .utils.logging import MetricsWriter
        self._metrics = MetricsWriter(path)
