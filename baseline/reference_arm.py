"""Reference arm of bench.py: the UNMODIFIED reference library (installed from its source tree into
baseline/_ref) trains the same Llama-style model through its own public Python API.

Nothing of litetorch_b200 is imported here.  The model is composed from the reference's stock ops
(`lt.Ops.matmul/add/mul/div/sqrt/sigmoid/softmax/rope/cat/cross_entropy_loss`, `lt.nn.Embedding`,
`lt.optim.AdamW`), because the reference has no RMSNorm, SwiGLU, causal or grouped-query attention op:
  RMSNorm      = x / sqrt(mean(x^2) + eps) * w      with mean(x^2) as a matmul against a constant column
  attention    = softmax(Q K^T * scale + causal mask) V on [B, H, T, T] scores (its flash_attention op has
                 no mask argument), KV heads repeated across the group with `Ops.cat`
  SwiGLU       = (g * sigmoid(g)) * u
The reference has no bf16 GEMM path on CUDA (bf16 tensors fall into the fp32 branch of Ops::matmul), so
this arm computes in fp32 (TF32 tensor cores are the reference's default for cublasSgemm).

A two-layer probe model is always trained and timed (key "probe": the same model bench.py's own arm times), so a
same-configuration ratio exists even when the full configuration cannot run.  The full configuration is first
projected from two layers at the 1.1B width under a wall-clock budget; when it cannot run (error, out of memory,
slower than the budget allows, more than one GPU) the line carries "unavailable": "<why>" and the arm exits 0.
"""
from __future__ import annotations

import json
import math
import os
import random
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")

# Wall-clock budget for the whole arm (seconds); one full-size step is projected from a probe first.
BUDGET_S = float(os.environ.get("LT_REFERENCE_BUDGET_S", "1500"))


def _unavailable(why: str):
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why[:300]}), flush=True)


class RefLlama:
    def __init__(self, lt, dev, V, L, D, Hq, Hkv, hd, F, T, B, theta=1e4, eps=1e-5, seed=0):
        self.lt, self.dev = lt, dev
        self.V, self.L, self.D, self.Hq, self.Hkv, self.hd, self.F, self.T, self.B = V, L, D, Hq, Hkv, hd, F, T, B
        rnd = random.Random(seed)
        import numpy as np
        rng = np.random.default_rng(seed)

        def P(shape, std=0.02):
            n = 1
            for s in shape:
                n *= s
            return lt.Tensor.from_vector(rng.normal(0.0, std, n).astype("float32").tolist(), list(shape), dev, True)

        def const(vals, shape, grad=False):
            return lt.Tensor.from_vector(vals, list(shape), dev, grad)

        self.emb = lt.nn.Embedding(V, D)
        self.emb.to(dev)
        self.emb.weight.copy_(P([V, D]))
        self.layers = []
        for _ in range(L):
            self.layers.append(dict(
                n1=const([1.0] * D, [D], True), n2=const([1.0] * D, [D], True),
                wq=P([D, Hq * hd]), wk=P([D, Hkv * hd]), wv=P([D, Hkv * hd]), wo=P([Hq * hd, D]),
                wg=P([D, F]), wu=P([D, F]), wd=P([F, D])))
        self.nf = const([1.0] * D, [D], True)
        self.head = P([D, V])
        self.mean_col = const([1.0 / D] * D, [D, 1])
        self.eps = const([eps], [1])
        self.scale = const([1.0 / math.sqrt(hd)], [1])
        cos, sin = [], []
        for t in range(T):
            for i in range(hd // 2):
                a = t / (theta ** (2 * i / hd))
                cos.append(math.cos(a))
                sin.append(math.sin(a))
        self.cos = const(cos, [T, hd // 2])
        self.sin = const(sin, [T, hd // 2])
        mask = np.triu(np.full((T, T), -1e9, dtype="float32"), k=1)
        self.mask = const(mask.reshape(-1).tolist(), [1, 1, T, T])

    def parameters(self):
        ps = [self.emb.weight, self.head, self.nf]
        for l in self.layers:
            ps += [l[k] for k in ("n1", "n2", "wq", "wk", "wv", "wo", "wg", "wu", "wd")]
        return ps

    def rms(self, x, w):
        O = self.lt.Ops
        ms = O.matmul(O.mul(x, x), self.mean_col)
        r = O.sqrt(O.add(ms, self.eps))
        return O.mul(O.div(x, r), w)

    def heads(self, x, H):
        return x.view([self.B, self.T, H, self.hd]).transpose(1, 2).contiguous()

    def forward(self, tok):
        O = self.lt.Ops
        G = self.Hq // self.Hkv
        x = self.emb.forward(tok)
        for l in self.layers:
            h = self.rms(x, l["n1"])
            q = O.rope(self.heads(O.matmul(h, l["wq"]), self.Hq), self.cos, self.sin)
            k = O.rope(self.heads(O.matmul(h, l["wk"]), self.Hkv), self.cos, self.sin)
            v = self.heads(O.matmul(h, l["wv"]), self.Hkv)
            if G > 1:
                k = O.cat([k] * G, 1)
                v = O.cat([v] * G, 1)
            s = O.matmul(q, k.transpose(2, 3).contiguous())
            s = O.add(O.mul(s, self.scale), self.mask)
            a = O.matmul(O.softmax(s, -1), v).transpose(1, 2).contiguous().view([self.B, self.T, self.Hq * self.hd])
            x = O.add(x, O.matmul(a, l["wo"]))
            h = self.rms(x, l["n2"])
            g = O.matmul(h, l["wg"])
            u = O.matmul(h, l["wu"])
            x = O.add(x, O.matmul(O.mul(O.mul(g, O.sigmoid(g)), u), l["wd"]))
        return O.matmul(self.rms(x, self.nf), self.head)


def _batch(lt, dev, V, B, T, rnd):
    seq = [[rnd.randrange(V) for _ in range(T + 1)] for _ in range(B)]
    tok = lt.Tensor.from_vector([float(s[t]) for s in seq for t in range(T)], [B, T], dev, False)
    tgt = lt.Tensor.from_vector([float(s[t + 1]) for s in seq for t in range(T)], [B * T], dev, False)
    return tok, tgt, B * T * 4 * 2


def _train_steps(lt, model, opt, dev, n, rnd, sync):
    times, losses, h2d = [], [], 0
    for _ in range(n):
        tok, tgt, nb = _batch(lt, dev, model.V, model.B, model.T, rnd)
        h2d = nb
        sync()
        t0 = time.perf_counter()
        opt.zero_grad()
        logits = model.forward(tok)
        loss = lt.Ops.cross_entropy_loss(logits.view([model.B * model.T, model.V]), tgt)
        loss.backward()
        opt.step()
        losses.append(loss.item())  # device -> host read, also the step's completion point
        times.append(time.perf_counter() - t0)
    return times, losses, h2d


TINY = (512, 2, 256, 4, 2, 64, 512)                 # vocab, layers, d, q heads, kv heads, head dim, ffn: bench.py's probe model
W1B = (32000, 22, 2048, 32, 4, 64, 5632)            # the 1.1B configuration
W8B = (128256, 32, 4096, 32, 8, 128, 14336)         # the Llama-3-8B shape of the headline


def _time_model(lt, dev, shape, layers, T, B, steps, warmup, sync, seed=1234):
    V, _, D, Hq, Hkv, hd, F = shape
    rnd = random.Random(seed)
    model = RefLlama(lt, dev, V, layers, D, Hq, Hkv, hd, F, T, B)
    opt = lt.optim.AdamW(model.parameters(), lr=3e-4, beta1=0.9, beta2=0.95, weight_decay=0.1)
    if warmup:
        _train_steps(lt, model, opt, dev, warmup, rnd, sync)
    times, losses, h2d = _train_steps(lt, model, opt, dev, steps, rnd, sync)
    del model, opt
    try:
        lt.empty_cache()
    except Exception:
        pass
    return times, losses, h2d


def run(args, micro_batch: int, seq_len: int):
    """Prints one JSON line.  The two-layer `probe` model (the same one bench.py's own arm reports under "probe") is
    always trained and timed, on one GPU, so that a same-configuration ratio exists; the full configuration is run
    only when a width probe shows that it fits the time budget, else the line says `unavailable` and why."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if int(os.environ.get("RANK", "0")) != 0:
        return                                         # the reference runs on one GPU (see below); other ranks have nothing to do
    if not os.path.isdir(REF):
        _unavailable("baseline/_ref is missing (pip install of the reference was not done on this machine)")
        return
    sys.path.insert(0, REF)
    t_start = time.time()
    try:
        import litetorch as lt
    except Exception as e:
        _unavailable("import of the reference failed: %r" % (e,))
        return
    try:
        if not lt.is_gpu_available():
            _unavailable("the reference found no GPU backend (liblitetorch_gpu.so not loadable or no device)")
            return
        dev = lt.auto_device()
        backend = lt.get_backend_name()
    except Exception as e:
        _unavailable("reference backend probe failed: %r" % (e,))
        return

    def sync():
        try:
            lt.distributed.ProcessGroup.get().sync_comm()
        except Exception:
            pass

    name = getattr(args, "model", "llama3-8b")
    out = {"impl": "reference"}
    # ---- the probe model: runs on the reference's stock CUDA path
    try:
        pt, pl, ph2d = _time_model(lt, dev, TINY, 2, 256, 4, 20, 5, sync)
        out["probe"] = {"model": "llama-tiny (vocab 512, 2 layers, d 256, 4q/2kv heads x 64, SwiGLU 512)", "n_gpus": 1,
                        "global_batch": 4, "seq_len": 256, "dtype": "fp32 (reference has no bf16 GEMM path)",
                        "value": round(4 * 256 * 20 / sum(pt), 2), "e2e_value": round(4 * 256 * 20 / sum(pt), 2), "unit": "tokens/s",
                        "ms_per_step": round(sum(pt) / 20 * 1e3, 3), "steps": 20, "warmup": 5, "final_loss": round(pl[-1], 4),
                        "timing": "host wall clock around each step ending in loss.item()", "backend": backend}
    except Exception as e:
        out["probe_error"] = repr(e)[:200]
    if name == "llama-tiny":
        p = out.get("probe")
        if p is None:
            _unavailable("reference failed on the probe model: %s" % out.get("probe_error"))
            return
        out.update({"metric": "train tokens/s", "value": p["value"], "unit": "tokens/s", "n_gpus": 1, "steps": 20, "warmup": 5,
                    "ms_per_step": p["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                    "dtype": p["dtype"], "data": "synthetic",
                    "config": {"model": "llama-tiny", "global_batch": 4, "seq_len": 256, "parallelism": "single", "backend": backend},
                    "e2e": {"value": p["value"], "unit": "tokens/s", "h2d_bytes_per_step": 4 * 257 * 4 * 2, "d2h_bytes_per_step": 4},
                    "gpu_launches": None})
        print(json.dumps(out), flush=True)
        return
    # ---- the full configuration: project its cost from two layers at the 1.1B width (the 8B layers are 5x larger)
    shape = W8B if name == "llama3-8b" else W1B
    T, B = (8192, 1) if name == "llama3-8b" else (seq_len, micro_batch)
    why = None
    try:
        if os.environ.get("LT_REFERENCE_WIDTH_PROBE", "1") != "0":
            wt, wl, _ = _time_model(lt, dev, W1B, 2, 2048, 4, 1, 0, sync)
            per_layer = wt[-1] / 2.0
            scale = 1.0 if shape is W1B else (shape[2] * (shape[3] + 2 * shape[4]) * shape[5] + shape[2] * shape[3] * shape[5]
                                              + 3 * shape[2] * shape[6]) / float(2048 * 2560 + 2048 * 2048 + 3 * 2048 * 5632)
            projected = per_layer * shape[1] * scale
            need = projected * (args.steps + args.warmup)
            fact = ("two layers at the 1.1B width (d 2048, seq 2048, batch 4, fp32: its only working CUDA GEMM dtype) took %.1f s "
                    "per step on this GPU (loss %.3f); the %s configuration has %d layers of %.1fx that size: about %.0f s per step, "
                    "%.0f s for %d+%d steps against a budget of %.0f s" % (wt[-1], wl[-1], name, shape[1], scale, projected, need,
                                                                          args.warmup, args.steps, BUDGET_S))
            if need > BUDGET_S - (time.time() - t_start):
                why = "reference too slow for the full configuration: " + fact
        else:
            why = "reference too slow for the full configuration (width probe skipped by LT_REFERENCE_WIDTH_PROBE=0)"
    except Exception as e:
        why = "reference failed on its own stock path at the 1.1B width: %r (backend %s)" % (e, backend)
    if world > 1:
        why = ((why + "; ") if why else "") + (
            "and it cannot use %d GPUs: NCCLBridge::init passes a pointer where ncclCommInitRank takes the 128-byte id by value "
            "(src/distributed/distributed.cpp:888-889), FSDP::fully_shard is not bound to Python, every process pins device 0 "
            "(src/backend/gpu_native/entrypoint.cu:90-94); measured on one GPU of this box instead" % world)
    if why is not None:
        out["unavailable"] = why[:900]
        print(json.dumps(out), flush=True)
        return
    try:
        times, losses, h2d = _time_model(lt, dev, shape, shape[1], T, B, args.steps, args.warmup, sync)
    except Exception as e:
        out["unavailable"] = "reference failed on its own stock path: %r (backend %s)" % (e, backend)
        print(json.dumps(out), flush=True)
        return
    total = sum(times)
    val = B * T * args.steps / total
    out.update({
        "metric": "train tokens/s", "value": round(val, 2), "unit": "tokens/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(total / args.steps * 1e3, 2),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp32 (reference has no bf16 GEMM path)",
        "data": "synthetic",
        "config": {"model": "%s composed from the reference's stock ops" % name, "global_batch": B, "seq_len": T,
                   "parallelism": "single", "backend": backend,
                   "timing": "host wall clock around each step ending in loss.item() (the reference exposes no events)"},
        "e2e": {"value": round(val, 2), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4},
        "gpu_launches": None, "final_loss": round(losses[-1], 4)})
    print(json.dumps(out), flush=True)
