"""Training throughput of the parallel decoder configurations (tokens/s, device-timed, max over ranks).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 \
        -m litetorch_b200.models.run_config --config tp8 [--tiny] [--steps 5] [--warmup 3]

  tp8    Llama-3-8B shape, tensor parallel over all ranks with sequence parallelism, seq 8192, 8 sequences per step
  ep8    MoE decoder (8 SwiGLU experts, top-2, capacity 1.25, aux 0.01), expert parallel over all ranks with
         data-parallel attention, seq 4096, micro-batch 2 per rank
  hybrid Llama-style 3B, TP2 x CP2 x PP2 (8 ranks), seq 32768 split by zigzag ring attention, 1F1B with 8 micro-batches
         of one sequence, activation checkpointing

`--tiny` runs the same parallel structure on a small shape (any even world size for tp8 / ep8; 8, 4 or 2 ranks for
hybrid, dropping axes).  Synthetic uniform-random tokens, N(0, 0.02) initialisation, AdamW (fp32 master weights).
One JSON line is printed by rank 0.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from ..core import Tensor, _unwrap
from ..optim import AdamW
from .decoder import PRESETS, ParallelDecoder, ParallelDims, shard_batch, tiny
from ..utils import sections
from ..utils.sections import section


def _make_groups(world: int, rank: int, tp: int, cp: int, pp: int, dp: int):
    """rank = ((pp_i * dp + dp_i) * cp + cp_i) * tp + tp_i; every rank creates every group, in the same order."""
    assert tp * cp * pp * dp == world
    coords = lambda r: (r // (dp * cp * tp), (r // (cp * tp)) % dp, (r // tp) % cp, r % tp)   # noqa: E731
    mine = coords(rank)
    out = {}
    for axis, name in ((3, "tp"), (2, "cp"), (1, "dp"), (0, "pp")):
        sizes = {"tp": tp, "cp": cp, "dp": dp, "pp": pp}
        if sizes[name] == 1:
            out[name] = None
            continue
        buckets = {}
        for r in range(world):
            c = coords(r)
            key = tuple(v for i, v in enumerate(c) if i != axis)
            buckets.setdefault(key, []).append(r)
        for key in sorted(buckets):
            g = dist.new_group(buckets[key])
            if rank in buckets[key]:
                out[name] = g
    return out, mine


class _Stage:
    """What PipelineParallelModule calls per micro-batch: token ids on the first stage, row activations elsewhere."""

    def __init__(self, model: ParallelDecoder, B: int, T_local: int):
        self.model, self.B, self.T = model, B, T_local

    def __call__(self, x: Tensor) -> Tensor:
        from ..core import _unwrap
        t = _unwrap(x)
        rows = self.model.embed_tokens(t) if self.model.is_first else t
        return Tensor(self.model.run_layers(rows, self.B, self.T))

    def parameters(self):
        return [Tensor(p) for p in self.model.parameters()]


def _parser():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", choices=["tp8", "ep8", "hybrid"], required=True)
    ap.add_argument("--tiny", action="store_true")
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-fused", action="store_true", help="plain NCCL collectives instead of the fused kernels")
    ap.add_argument("--seq", type=int, default=0)
    ap.add_argument("--n-seq", type=int, default=0, help="sequences per micro-batch (default: the layout's)")
    ap.add_argument("--fp8", action="store_true", help="e4m3 GEMMs with 1x128 / 128x128 block scales (NCCL collectives)")
    ap.add_argument("--layout", default="", help="hybrid only: tp,cp,pp sizes (e.g. 1,2,2) instead of the default for the world size")
    ap.add_argument("--micro", type=int, default=0, help="micro-batches per step (default: the layout's)")
    ap.add_argument("--cp-mode", choices=["ring", "ulysses"], default="ring",
                    help="context parallelism: all-ranks ring attention (zigzag split) or Ulysses all-to-all (contiguous split)")
    return ap


def main():
    run(_parser().parse_args())


def run(args, quiet: bool = False):
    """Runs one configuration (`args`: the namespace of `_parser()`) and returns its result record (rank 0 also prints it unless `quiet`).  When the
    process group already exists (a caller that measures several configurations in one job) it is used and left
    alive; otherwise it is created here and destroyed at the end."""
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    cuda = torch.cuda.is_available()
    if cuda:
        torch.cuda.set_device(local)
    dev = "cuda" if cuda else "cpu"
    own_pg = not dist.is_initialized()
    if own_pg:
        dist.init_process_group("nccl" if cuda else "gloo", rank=rank, world_size=world,
                                device_id=torch.device("cuda", local) if cuda else None)
    dtype = torch.bfloat16 if cuda else torch.float32
    fused = cuda and not args.no_fused and world > 1

    if args.config == "tp8":
        cfg = PRESETS["tiny-dense"] if args.tiny else PRESETS["llama3-8b"]
        seq = args.seq or (512 if args.tiny else 8192)
        n_seq, micro = (2 if args.tiny else 8), 1
        groups, _ = _make_groups(world, rank, world, 1, 1, 1)
        layout = "tp%d+sp" % world
    elif args.config == "ep8":
        cfg = PRESETS["tiny-moe"] if args.tiny else PRESETS["moe-8x2b"]
        if cfg.n_experts % world:
            cfg = tiny(cfg, n_experts=world * max(1, cfg.n_experts // world))
        seq = args.seq or (256 if args.tiny else 4096)
        n_seq, micro = 2, 1
        groups = {"tp": None, "cp": None, "pp": None, "dp": None}
        layout = "ep%d+dp-attention" % world
    else:
        cfg = PRESETS["tiny-dense"] if args.tiny else PRESETS["llama-3b-long"]
        seq = args.seq or (1024 if args.tiny else 32768)
        n_seq, micro = 1, 8
        tp, cp, pp = (2, 2, 2) if world >= 8 else ((2, 2, 1) if world == 4 else ((2, 1, 1) if world == 2 else (1, 1, 1)))
        if args.layout:
            tp, cp, pp = (int(v) for v in args.layout.split(","))
        groups, _ = _make_groups(world, rank, tp, cp, pp, world // (tp * cp * pp))
        layout = "tp%d x cp%d x pp%d" % (tp, cp, pp)
    if args.n_seq:
        n_seq = args.n_seq
    if args.micro:
        micro = args.micro
    ep_group = dist.group.WORLD if (args.config == "ep8" and world > 1) else None

    dims = ParallelDims(tp=groups["tp"], cp=groups["cp"], ep=ep_group, dp=groups["dp"], pp=groups["pp"], zigzag=True,
                        fp8=args.fp8 and cuda, cp_mode=args.cp_mode)
    T_local = seq // dims.cp_world
    hq_l, hkv_l = cfg.n_q // dims.tp_world, cfg.n_kv // dims.tp_world
    if fused and dims.tp is not None:
        from ..parallel.tp_fused import TPFusedContext
        # gathered inputs and scattered outputs of the parallel linears are all d_model wide
        dims.tp_fused = TPFusedContext(n_seq * T_local, cfg.d_model, dev, group=dims.tp)
    if fused and dims.cp is not None and dims.cp_mode == "ring":
        from ..parallel.cp import RingFlashContext
        dims.cp_fused = RingFlashContext(n_seq, T_local, hq_l, hkv_l, cfg.head_dim, dev, group=dims.cp, zigzag=True)

    pp_world = dist.get_world_size(groups["pp"]) if groups["pp"] is not None else 1
    pp_rank = dist.get_rank(groups["pp"]) if groups["pp"] is not None else 0
    per = cfg.n_layers // pp_world
    model = ParallelDecoder(cfg, dims, device=dev, dtype=dtype, seed=1, first_layer=pp_rank * per,
                            last_layer=(pp_rank + 1) * per if pp_rank < pp_world - 1 else cfg.n_layers,
                            max_tokens=n_seq * T_local, activation_checkpointing=(args.config == "hybrid"))
    opt = AdamW([Tensor(p) for p in model.parameters()], lr=3e-4, beta1=0.9, beta2=0.95, weight_decay=0.1)

    gen = torch.Generator().manual_seed(1234 + (0 if args.config != "ep8" else rank))
    def batch():
        ids = torch.randint(0, cfg.vocab, (n_seq, seq + 1), generator=gen)
        x, y = ids[:, :-1], ids[:, 1:]
        return shard_batch(x, dims).to(dev), shard_batch(y, dims).to(dev)

    pipe = None
    if pp_world > 1:
        from ..parallel.pp import PipelineParallelModule
        pipe = PipelineParallelModule(_Stage(model, n_seq, T_local), group=groups["pp"], device=dev)

    def step():
        opt.zero_grad()
        if pipe is None:
            for _ in range(micro):
                x, y = batch()
                with section("step.forward"):
                    loss = model.forward_loss(x, y)
                with section("step.backward"):
                    (loss / micro).backward()
            last = loss.detach()
        else:
            mbs = [batch() for _ in range(micro)]
            xs, ys = [Tensor(m[0]) for m in mbs], [m[1] for m in mbs]
            val = pipe.train_step_1f1b(xs, lambda out, tgt: Tensor(model.loss(_unwrap(out), tgt)), ys)
            last = torch.tensor(val, device=dev)
        with section("step.reduce_gradients"):
            model.reduce_gradients()
        with section("step.optimizer"):
            opt.step()
        return last

    # Bring the ranks together before the first step: every group's communicator is created by a first small collective
    # here rather than inside the step, where seconds of skew between ranks would meet the bounded waits of the fused kernels.
    for g in list(groups.values()) + [ep_group, None]:
        if g is not None or world > 1:
            dist.all_reduce(torch.zeros(1, device=dev), group=g)
    if cuda:
        torch.cuda.synchronize()
    dist.barrier()
    for _ in range(args.warmup):
        last = step()
    sections.reset()
    if cuda:
        torch.cuda.synchronize()
    dist.barrier()
    if cuda:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
    import time
    t0 = time.perf_counter()
    for _ in range(args.steps):
        last = step()
    if cuda:
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / args.steps
    else:
        ms = (time.perf_counter() - t0) * 1e3 / args.steps
    t = torch.tensor([ms], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    # the last pipeline stage holds the loss (0.0 elsewhere); a NaN must not be hidden by the maximum
    lv = torch.nan_to_num(last.float().reshape(1).clone(), nan=float("inf"))
    # every rank's loss is the mean over its own tokens: average over the ranks that hold other tokens of the same step
    # (context- and data-parallel groups; all ranks in the expert-parallel layout), then take the last stage's value
    for g in ([dist.group.WORLD] if (args.config == "ep8" and world > 1) else [groups["cp"], groups["dp"]]):
        if g is not None and dist.get_world_size(g) > 1:
            dist.all_reduce(lv, group=g)
            lv /= dist.get_world_size(g)
    dist.all_reduce(lv, op=dist.ReduceOp.MAX)
    dp_like = world if args.config == "ep8" else (dist.get_world_size(groups["dp"]) if groups["dp"] is not None else 1)
    tokens = n_seq * seq * micro * dp_like
    status = 0
    if cuda:
        from ..ops import kernels as K
        st = torch.tensor([K.status_fetch()], device=dev)
        dist.all_reduce(st, op=dist.ReduceOp.MAX)
        status = int(st)
    record = {"config": args.config, "model": cfg.name, "layout": layout, "n_gpus": world, "seq_len": seq,
              "tokens_per_step": tokens, "ms_per_step": round(float(t), 3),
              "tokens_per_s": round(tokens / float(t) * 1e3, 1), "loss": round(float(lv), 4),
              "fused": bool(fused) and not dims.fp8, "fp8": bool(dims.fp8), "dtype": str(dtype).replace("torch.", ""),
              "device_status": status, "params_b": round(cfg.n_params() / 1e9, 3), "steps": args.steps, "warmup": args.warmup}
    if rank == 0 and not quiet:
        print(json.dumps(record), flush=True)
    if rank == 0 and sections.enabled():
        # per-section CUDA-event totals over the timed steps (LT_SECTIONS=1); nested sections are included in their parents
        print(json.dumps({"sections_ms_per_step": {k: [v[0] // max(args.steps, 1), round(v[1] / max(args.steps, 1), 3)]
                                                   for k, v in sections.report().items()}}), flush=True)
    dist.barrier()
    if own_pg:
        dist.destroy_process_group()
    return record


if __name__ == "__main__":
    main()
