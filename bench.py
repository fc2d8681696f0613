#!/usr/bin/env python
"""Headline benchmark: training tokens/s of the Llama-3-8B shape (vocab 128256, 32 layers, d 4096, 32 q / 8 kv heads
of 128, SwiGLU 14336, RoPE 5e5, seq 8192, one sequence per GPU and step, bf16 compute, fp32 master + AdamW states)
under FSDP (ZeRO-3) x tensor parallelism with sequence parallelism on N GPUs of one node (weak scaling: tokens per
GPU are fixed).  Mesh per N (dp x tp): 1 -> 1x1, 2 -> 1x2, 4 -> 2x2, 8 -> 4x2: tensor parallelism stays inside a pair
of GPUs, where the fused all-gather -> GEMM / GEMM -> reduce-scatter kernels run near their roofline, and the other
ranks shard parameters, gradients and optimizer state the ZeRO-3 way (`--tp` changes the split).

    python bench.py --gpus 1 --steps 10 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 \
        bench.py --gpus 8 --steps 10 --warmup 3
    python bench.py --impl reference ...      # the unmodified reference library from baseline/_ref

Rank 0 prints ONE JSON line.  `value` is device-timed (CUDA events around exactly K steps, barrier +
synchronize on both sides, max over ranks) with batches already on the device; `e2e` times the public
`Trainer.step` call, which copies each batch from pinned host memory and reads the loss back every step.
Outside the timed regions the line also carries: `exposed_comm_ms_per_step` (the step minus the same per-GPU
compute without any communication), `llama_1b` (the 1.1B ZeRO-3 configuration: vocab 32000, 22 layers, d 2048,
seq 2048, micro-batch 4 per GPU) and `probe` (a two-layer model small enough for the reference library to train,
for a same-configuration ratio).  Data are synthetic uniform-random tokens, weights N(0, 0.02).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

# name -> (sequences per GPU and step, sequence length)
SHAPES = {"llama3-8b": (1, 8192), "llama-1.1b": (4, 2048), "llama-tiny": (4, 256)}
MICRO_BATCH = 4          # of the 1.1B configuration and of the probe (the reference arm uses the same)
SEQ_LEN = 2048


def _parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="llama3-8b", choices=list(SHAPES))
    ap.add_argument("--tp", type=int, default=0, help="tensor-parallel size (0: 1 on one GPU, else 2)")
    ap.add_argument("--ckpt", default="auto",
                    help="activation checkpointing: auto (as many layers as the memory of one rank needs), on, off, "
                         "or the number of layers whose activations are recomputed in the backward pass")
    ap.add_argument("--no-comm-breakdown", action="store_true",
                    help="skip the extra communication-free steps that give exposed_comm_ms_per_step at N > 1")
    ap.add_argument("--no-extras", action="store_true", help="skip the llama_1b and probe measurements")
    ap.add_argument("--configs", default="auto", choices=["auto", "on", "off"],
                    help="also time the three other 8-GPU layouts (tp8, ep8, tp2 x cp2 x pp2) outside the timed region "
                         "(auto: on 8 GPUs)")
    ap.add_argument("--hybrid", action="store_true",
                    help="with --tp 1: shard over dp with the FSDP x TP provider (weights prefetched by peer-pull kernels) "
                         "instead of the ZeRO-3 provider whose all-gather runs inside the GEMMs")
    return ap.parse_args()


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples taken while the timed region runs (read-only queries)."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(prefix="lt_clocks_", suffix=".csv")
            os.close(fd)
            self.f = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu), "--query-gpu=" + self.FIELDS,
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=self.f,
                                         stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        try:
            self.proc.terminate()
            self.proc.wait(timeout=5)
        except Exception:
            try:
                self.proc.kill()
            except Exception:
                pass
        try:
            self.f.close()
            sm, reasons, mx, pw = [], set(), None, []
            names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
            with open(self.path) as f:
                for line in f:
                    parts = [p.strip() for p in line.split(",")]
                    if len(parts) < 9:
                        continue
                    try:
                        sm.append(float(parts[1]))
                        mx = float(parts[2])
                        pw.append(float(parts[3]))
                    except ValueError:
                        continue
                    for n, v in zip(names, parts[5:9]):
                        if v.lower().startswith("active"):
                            reasons.add(n)
            os.unlink(self.path)
            if sm:
                # keep the samples taken under load (upper half by power) for the median
                sm_sorted = sorted(sm)
                out = {"sm_mhz": sm_sorted[len(sm_sorted) // 2], "sm_max_mhz": mx, "reasons": sorted(reasons),
                       "samples": len(sm), "power_w_max": max(pw) if pw else None}
        except Exception:
            pass
        return out


def _model_config(name):
    from litetorch_b200.models.llama import LlamaConfig
    return {"llama3-8b": LlamaConfig.llama3_8b, "llama-1.1b": LlamaConfig.llama_1b, "llama-tiny": LlamaConfig.tiny}[name]()


def _describe(cfg):
    return "%s (vocab %d, %d layers, d %d, %dq/%dkv heads x %d, SwiGLU %d, RMSNorm, RoPE %g)" % (
        cfg.name, cfg.vocab_size, cfg.n_layers, cfg.d_model, cfg.n_heads, cfg.n_kv_heads, cfg.head_dim, cfg.ffn, cfg.rope_theta)


def _measure(tr, host, devb, steps, warmup, sync, sampler=None):
    """Device-timed steps on resident batches, then the same number end to end through Trainer.step.
    Returns (ms_total, e2e_ms_total, launches, last loss, clocks)."""
    import torch
    from litetorch_b200.ops import kernels as K
    n = len(devb)
    for i in range(warmup):
        tr.step_device(*devb[i % n])
    sync()
    if sampler is not None:
        sampler.start()
    K.reset_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync()
    e0.record()
    last = None
    for i in range(steps):
        last = tr.step_device(*devb[i % n])
    e1.record()
    sync()
    launches = K.launch_count()
    ms_total = e0.elapsed_time(e1)
    clocks = sampler.stop() if sampler is not None else {}
    loss_val = float(last)
    for i in range(warmup):
        tr.step(*host[i % n])
    sync()
    t0 = time.perf_counter()
    for i in range(steps):
        tr.step(*host[i % n])
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3
    sync()
    return ms_total, e2e_ms, launches, loss_val, clocks


def _batches(cfg, n_seq, T, seed, dev, n_batches=4):
    import torch
    gen = torch.Generator(device="cpu").manual_seed(seed)
    host = []
    for _ in range(n_batches):
        seq = torch.randint(0, cfg.vocab_size, (n_seq, T + 1), generator=gen, dtype=torch.int64)
        host.append((seq[:, :-1].contiguous().pin_memory(), seq[:, 1:].contiguous().pin_memory()))
    return host, [(a.to(dev), b.to(dev)) for a, b in host]


def run_ours(args):
    import dataclasses
    import torch
    import torch.distributed as dist
    from litetorch_b200.ops import kernels as K
    from litetorch_b200.trainer import Trainer

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1 and not dist.is_initialized():
        # NCCL carries only small messages here (norm-gain gradients, cross-entropy statistics, one embedding-gradient
        # gather); in-switch reduction is left off so that no rank's memory is bound to a multicast object
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=dev)
    cfg = _model_config(args.model)
    per_gpu, T = SHAPES[args.model]
    T = min(T, cfg.max_seq)
    big = args.model == "llama3-8b"
    tp = args.tp or int(os.environ.get("LT_BENCH_TP", "0")) or (2 if (world > 1 and big) else 1)
    dp = world // tp
    if args.ckpt == "auto":
        ckpt = 0        # 8B on one GPU: 156 GB peak of 180 GB without recomputation (falls back to full recomputation if it does not fit)
    else:
        ckpt = {"on": cfg.n_layers, "off": 0}.get(args.ckpt, None)
        ckpt = int(args.ckpt) if ckpt is None else ckpt
    n_seq = per_gpu * tp                           # sequences of one tensor-parallel group (all its ranks get the same batch)

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    host, devb = _batches(cfg, n_seq, T, 1000 + rank // tp, dev)
    sampler = ClockSampler(local) if rank == 0 else None
    try:
        tr = Trainer(cfg, seed=1234, tp=tp, activation_checkpointing=ckpt, parallel="hybrid" if (tp > 1 or args.hybrid) else "auto")
        ms_total, e2e_ms, launches, loss_val, clocks = _measure(tr, host, devb, args.steps, args.warmup, sync, sampler)
    except torch.cuda.OutOfMemoryError:
        # Single GPU only (no peer is left waiting): saved activations did not fit beside 128 GB of weights and
        # optimizer state on this device, so recompute every layer in the backward pass instead.
        if world > 1 or ckpt == cfg.n_layers:
            raise
        if sampler is not None:
            sampler.stop()
        tr = None
        import gc
        gc.collect()
        torch.cuda.empty_cache()
        ckpt = cfg.n_layers
        tr = Trainer(cfg, seed=1234, tp=tp, activation_checkpointing=ckpt)
        ms_total, e2e_ms, launches, loss_val, clocks = _measure(tr, host, devb, args.steps, args.warmup, sync, sampler)
    h2d_bytes, d2h_bytes = tr.h2d_bytes, tr.d2h_bytes
    status = K.status_fetch()
    peak_gb = torch.cuda.max_memory_allocated() / 2 ** 30
    del tr
    torch.cuda.empty_cache()

    # ---------------- exposed communication (outside the timed regions): the same per-GPU compute with no
    # communication at all.  For the ZeRO-3 layout that is an unsharded copy of the model on each GPU; for a
    # tensor-parallel group it is the group's batch through a model whose heads, feed-forward width and vocabulary
    # are divided by tp (exactly the GEMM / attention shapes one rank executes).  What the sharded step takes on top
    # of it is communication that the overlap did not hide (gather CTAs taken from the GEMMs included).
    local_ms = 0.0
    if world > 1 and not args.no_comm_breakdown:
        twin = dataclasses.replace(cfg, n_heads=cfg.n_heads // tp, n_kv_heads=cfg.n_kv_heads // tp, ffn=cfg.ffn // tp,
                                   vocab_size=cfg.vocab_size // tp)
        tr_local = Trainer(twin, seed=1234, parallel="none", activation_checkpointing=ckpt)
        _, tb = _batches(twin, n_seq, T, 1000 + rank // tp, dev)
        for i in range(3):
            tr_local.step_device(*tb[i % len(tb)])
        torch.cuda.synchronize()
        l0, l1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        l0.record()
        for i in range(4):
            tr_local.step_device(*tb[i % len(tb)])
        l1.record()
        torch.cuda.synchronize()
        local_ms = l0.elapsed_time(l1) / 4
        del tr_local, tb
        torch.cuda.empty_cache()

    # ---------------- extras, outside the timed regions
    extras = {}
    if not args.no_extras and big:
        try:
            c1 = _model_config("llama-1.1b")
            b1, t1 = SHAPES["llama-1.1b"]
            tr1 = Trainer(c1, seed=1234)
            h1, d1 = _batches(c1, b1, t1, 2000 + rank, dev)
            ms1, e2e1, _, loss1, _ = _measure(tr1, h1, d1, 6, 3, sync)
            loc1 = 0.0
            del tr1
            torch.cuda.empty_cache()
            if world > 1:
                tl = Trainer(c1, seed=1234, parallel="none")
                for i in range(3):
                    tl.step_device(*d1[i % len(d1)])
                torch.cuda.synchronize()
                l0, l1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                l0.record()
                for i in range(4):
                    tl.step_device(*d1[i % len(d1)])
                l1.record()
                torch.cuda.synchronize()
                loc1 = l0.elapsed_time(l1) / 4
                del tl
                torch.cuda.empty_cache()
            extras["llama_1b"] = (ms1, e2e1, loc1, loss1)
        except Exception as e:  # pragma: no cover
            extras["llama_1b_error"] = repr(e)[:200]
        try:
            cp_ = _model_config("llama-tiny")
            bp, tpb = SHAPES["llama-tiny"]
            trp = Trainer(cp_, seed=1234, parallel="none")
            hp, dpb = _batches(cp_, bp, tpb, 3000, dev)
            msp, e2ep, _, lossp, _ = _measure(trp, hp, dpb, 20, 5, lambda: torch.cuda.synchronize())
            extras["probe"] = (msp, e2ep, lossp)
            del trp
        except Exception as e:  # pragma: no cover
            extras["probe_error"] = repr(e)[:200]

    # ---------------- the other multi-GPU layouts (8 GPUs), outside the timed regions, under a wall-clock limit: when it
    # runs out the line is printed without them (a stuck collective must not take the headline with it)
    want_cfgs = (args.configs == "on") or (args.configs == "auto" and world == 8 and big and not args.no_extras)
    state = {"partial": None}
    if want_cfgs and world > 1:
        import threading
        limit = float(os.environ.get("LT_BENCH_CONFIGS_LIMIT_S", "420"))

        def give_up():
            if rank == 0 and state["partial"] is not None:
                line = dict(state["partial"])
                line["configs"] = dict(state.get("configs", {}), error="time limit of %.0f s reached" % limit)
                print(json.dumps(line), flush=True)
            os._exit(0)

        timer = threading.Timer(limit, give_up)
        timer.daemon = True
    else:
        timer = None

    vals = [ms_total, e2e_ms, local_ms]
    if "llama_1b" in extras:
        vals += list(extras["llama_1b"][:3])
    t = torch.tensor(vals, device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total, e2e_ms, local_ms = float(t[0]), float(t[1]), float(t[2])
    tokens = per_gpu * T * world * args.steps
    value = tokens / (ms_total / 1e3)
    e2e_value = tokens / (e2e_ms / 1e3)
    if rank == 0:
        par = "single" if world == 1 else ("fsdp%d (ZeRO-3)" % world if tp == 1 else
                                            "dp%d (ZeRO-3) x tp%d (+ sequence parallel)" % (dp, tp))
        out = {
            "metric": "train tokens/s", "value": round(value, 1), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_total / args.steps, 3),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "impl": "ours",
            "config": {"model": _describe(cfg), "global_batch": per_gpu * world, "seq_len": T, "parallelism": par,
                       "dp": dp, "tp": tp, "checkpointed_layers": int(ckpt),
                       "optimizer": "AdamW fp32 master+states, bf16 params/grads",
                       "l2": "no flush: the step's working set (weights and activations, tens of GB) is far larger than the 126 MB L2"},
            "clocks": clocks,
            "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s", "ms_per_step": round(e2e_ms / args.steps, 3),
                    "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": d2h_bytes},
            "gpu_launches": launches,
            "exposed_comm_ms_per_step": (round(ms_total / args.steps - local_ms, 3) if local_ms > 0 else (0.0 if world == 1 else None)),
            "comm_free_step_ms": round(local_ms, 3) if local_ms > 0 else None,
            "final_loss": round(loss_val, 4),
            "device_status": status,
            "peak_memory_gb": round(peak_gb, 1),
            "model_tflops_per_gpu": round(cfg.flops_per_token(T) * value / world / 1e12, 1),
        }
        if "llama_1b" in extras:
            ms1, e2e1, loc1 = float(t[3]), float(t[4]), float(t[5])
            tok1 = SHAPES["llama-1.1b"][0] * SHAPES["llama-1.1b"][1] * world
            out["llama_1b"] = {"value": round(tok1 * 6 / (ms1 / 1e3), 1), "unit": "tokens/s", "ms_per_step": round(ms1 / 6, 3),
                               "e2e_value": round(tok1 * 6 / (e2e1 / 1e3), 1),
                               "exposed_comm_ms_per_step": round(ms1 / 6 - loc1, 3) if loc1 > 0 else 0.0,
                               "parallelism": "single" if world == 1 else "fsdp%d (ZeRO-3)" % world,
                               "global_batch": SHAPES["llama-1.1b"][0] * world, "seq_len": SHAPES["llama-1.1b"][1],
                               "steps": 6, "warmup": 3, "final_loss": round(extras["llama_1b"][3], 4)}
        if "probe" in extras:
            msp, e2ep, lossp = extras["probe"]
            tokp = SHAPES["llama-tiny"][0] * SHAPES["llama-tiny"][1]
            out["probe"] = {"model": "llama-tiny (vocab 512, 2 layers, d 256, 4q/2kv heads x 64, SwiGLU 512)", "n_gpus": 1,
                            "global_batch": SHAPES["llama-tiny"][0], "seq_len": SHAPES["llama-tiny"][1], "dtype": "bf16",
                            "value": round(tokp * 20 / (msp / 1e3), 1), "e2e_value": round(tokp * 20 / (e2ep / 1e3), 1),
                            "unit": "tokens/s", "ms_per_step": round(msp / 20, 4), "steps": 20, "warmup": 5,
                            "final_loss": round(lossp, 4)}
        for k in ("llama_1b_error", "probe_error"):
            if k in extras:
                out[k] = extras[k]
        state["partial"] = out
    if timer is not None:
        from litetorch_b200.models import run_config
        timer.start()
        cfgs = state.setdefault("configs", {})
        tiny = ["--tiny"] if not big else []
        for name in ("tp8", "ep8", "hybrid"):
            if name == "hybrid" and world not in (2, 4, 8):
                continue
            try:
                ns = run_config._parser().parse_args(["--config", name, "--steps", "3", "--warmup", "2"] + tiny)
                rec = run_config.run(ns, quiet=True)
                cfgs[name] = {k: rec[k] for k in ("model", "layout", "seq_len", "tokens_per_step", "ms_per_step", "tokens_per_s",
                                                  "loss", "fused", "device_status", "params_b", "steps", "warmup")}
            except Exception as e:  # pragma: no cover
                cfgs[name] = {"error": repr(e)[:200]}
            import gc
            gc.collect()
            torch.cuda.empty_cache()
        timer.cancel()
        if rank == 0:
            out["configs"] = cfgs
    if rank == 0:
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_reference(args):
    here = os.path.dirname(os.path.abspath(__file__))
    sys.path.insert(0, os.path.join(here, "baseline"))
    try:
        import reference_arm
    except Exception as e:  # pragma: no cover
        if int(os.environ.get("RANK", "0")) == 0:
            print(json.dumps({"impl": "reference", "unavailable": "reference arm not importable: %s" % str(e)[:160]}))
        return
    reference_arm.run(args, MICRO_BATCH, SEQ_LEN)


if __name__ == "__main__":
    a = _parse()
    if a.impl == "reference":
        run_reference(a)
    else:
        run_ours(a)
