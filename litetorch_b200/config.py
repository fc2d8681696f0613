"""Run configuration: model shape, parallel mesh, precision and schedule as dataclasses, loadable from JSON with
environment overrides, plus the five benchmark configurations as presets.

The reference has no configuration system: constructor arguments, a few environment variables and compile-time
macros (python/litetorch/__init__.py, src/core/backend.cpp:351-359).  Here one `RunConfig` describes a job:

    cfg = lt.config.load("llama-1.1b-fsdp")           # a preset name ...
    cfg = lt.config.load("job.json")                   # ... or a JSON file with the same fields
    LT_CFG_PARALLEL__TP=4 LT_CFG_SEQ_LEN=4096 python train.py     # environment overrides, `__` descends into a section

`RunConfig.mesh_sizes(world)` checks the mesh against the world size; `decoder_config()` / `llama_config()` build the
model-side dataclasses of `models/decoder.py` and `models/llama.py`.
"""
from __future__ import annotations

import json
import os
from dataclasses import asdict, dataclass, field, fields, is_dataclass
from typing import Any, Dict, Optional


@dataclass
class ModelConfig:
    name: str = "llama-1.1b"
    vocab: int = 32000
    n_layers: int = 22
    d_model: int = 2048
    n_q: int = 32
    n_kv: int = 4
    head_dim: int = 64
    ffn: int = 5632
    n_experts: int = 0              # 0: dense SwiGLU feed-forward
    top_k: int = 2
    capacity_factor: float = 1.25
    aux_loss_coef: float = 0.01
    rope_theta: float = 1e4
    eps: float = 1e-5
    norm: str = "rms"               # "rms" | "layer" (the CPU GPT configuration uses pre-LayerNorm + GELU)
    activation: str = "swiglu"      # "swiglu" | "gelu"


@dataclass
class ParallelConfig:
    dp: int = 0                     # 0: whatever is left of the world size after the other axes
    tp: int = 1
    pp: int = 1
    cp: int = 1
    ep: int = 1
    sequence_parallel: bool = True
    zero_stage: int = 3             # sharding of weights / gradients / optimizer states over dp (0 = replicated)
    cp_mode: str = "ring"           # "ring" (zigzag all-ranks attention) | "ulysses"
    fused: bool = True              # fused compute + collective kernels (False: NCCL collectives)


@dataclass
class OptimConfig:
    lr: float = 3e-4
    beta1: float = 0.9
    beta2: float = 0.95
    eps: float = 1e-8
    weight_decay: float = 0.1
    grad_clip: float = 0.0


@dataclass
class RunConfig:
    model: ModelConfig = field(default_factory=ModelConfig)
    parallel: ParallelConfig = field(default_factory=ParallelConfig)
    optim: OptimConfig = field(default_factory=OptimConfig)
    seq_len: int = 2048
    micro_batch: int = 4            # sequences per micro-batch per data-parallel rank
    micro_batches: int = 1          # micro-batches per step (pipeline schedule / gradient accumulation)
    precision: str = "bf16"         # "bf16" | "fp8" (e4m3 GEMMs, 1x128 / 128x128 block scales) | "fp32"
    activation_checkpointing: bool = False
    steps: int = 20
    seed: int = 0
    device: str = "cuda"

    # ---- (de)serialisation
    def to_dict(self) -> Dict[str, Any]:
        return asdict(self)

    def to_json(self, path: Optional[str] = None) -> str:
        text = json.dumps(self.to_dict(), indent=2, sort_keys=True)
        if path:
            with open(path, "w") as f:
                f.write(text + "\n")
        return text

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "RunConfig":
        return _build(cls, d, "")

    # ---- derived
    def mesh_sizes(self, world: int) -> Dict[str, int]:
        """Sizes of the dp / tp / pp / cp axes for `world` ranks (expert parallelism reuses the data-parallel ranks)."""
        p = self.parallel
        denom = p.tp * p.pp * p.cp
        if world % denom:
            raise ValueError("world size %d is not a multiple of tp*pp*cp = %d" % (world, denom))
        dp = p.dp or world // denom
        if dp * denom != world:
            raise ValueError("dp*tp*pp*cp = %d does not match the world size %d" % (dp * denom, world))
        if p.ep > 1 and (dp * p.cp) % p.ep and world % p.ep:
            raise ValueError("expert parallel size %d does not divide the ranks that hold a replica" % p.ep)
        m = self.model
        if m.n_q % p.tp or (m.n_kv % p.tp and p.tp % m.n_kv) or m.ffn % p.tp or m.n_layers % p.pp:
            raise ValueError("heads / ffn / layers do not divide over tp=%d pp=%d" % (p.tp, p.pp))
        if m.n_experts and m.n_experts % max(p.ep, 1):
            raise ValueError("experts do not divide over ep=%d" % p.ep)
        return {"dp": dp, "tp": p.tp, "pp": p.pp, "cp": p.cp, "ep": p.ep}

    def tokens_per_step(self, world: int) -> int:
        s = self.mesh_sizes(world)
        return self.seq_len * self.micro_batch * self.micro_batches * s["dp"]

    def decoder_config(self):
        from .models.decoder import DecoderConfig
        m = self.model
        return DecoderConfig(m.name, m.vocab, m.n_layers, m.d_model, m.n_q, m.n_kv, m.head_dim, m.ffn, rope_theta=m.rope_theta,
                             eps=m.eps, n_experts=m.n_experts, top_k=m.top_k, capacity_factor=m.capacity_factor,
                             aux_coef=m.aux_loss_coef)

    def llama_config(self):
        from .models.llama import LlamaConfig
        m = self.model
        return LlamaConfig(vocab_size=m.vocab, n_layers=m.n_layers, d_model=m.d_model, n_heads=m.n_q, n_kv_heads=m.n_kv,
                           head_dim=m.head_dim, ffn=m.ffn, rms_eps=m.eps, rope_theta=m.rope_theta, max_seq=self.seq_len,
                           name=m.name)


def _coerce(tp, v):
    if isinstance(v, str) and tp is not str:
        if tp is bool:
            return v.strip().lower() in ("1", "true", "yes", "on")
        return tp(v)
    if tp is float and isinstance(v, int):
        return float(v)
    return v


def _build(cls, d: Dict[str, Any], where: str):
    known = {f.name: f for f in fields(cls)}
    unknown = set(d) - set(known)
    if unknown:
        raise KeyError("unknown configuration field(s) %s%s" % (where, sorted(unknown)))
    kw = {}
    for name, f in known.items():
        if name not in d:
            continue
        default = getattr(cls(), name)
        if is_dataclass(default):
            kw[name] = _build(type(default), d[name], where + name + ".")
        else:
            kw[name] = _coerce(type(default), d[name])
    return cls(**kw)


def apply_env(cfg: RunConfig, env=None, prefix: str = "LT_CFG_") -> RunConfig:
    """`LT_CFG_SEQ_LEN=4096`, `LT_CFG_PARALLEL__TP=4`, `LT_CFG_MODEL__N_LAYERS=2`: top-level field or SECTION__FIELD."""
    env = os.environ if env is None else env
    for key, val in env.items():
        if not key.startswith(prefix):
            continue
        path = key[len(prefix):].lower().split("__")
        obj = cfg
        for part in path[:-1]:
            if not hasattr(obj, part) or not is_dataclass(getattr(obj, part)):
                raise KeyError("no configuration section %r (from %s)" % (part, key))
            obj = getattr(obj, part)
        leaf = path[-1]
        if not hasattr(obj, leaf) or is_dataclass(getattr(obj, leaf)):
            raise KeyError("no configuration field %r (from %s)" % (leaf, key))
        setattr(obj, leaf, _coerce(type(getattr(obj, leaf)), val))
    return cfg


def _presets() -> Dict[str, RunConfig]:
    gpt = RunConfig(model=ModelConfig("gpt-cpu", 256, 2, 128, 4, 4, 32, 512, norm="layer", activation="gelu"),
                    parallel=ParallelConfig(zero_stage=0, fused=False), seq_len=64, micro_batch=8, precision="fp32",
                    steps=20, device="cpu")
    llama1b = RunConfig()                                                   # the dataclass defaults are this configuration
    llama8b = RunConfig(model=ModelConfig("llama3-8b", 128256, 32, 4096, 32, 8, 128, 14336, rope_theta=5e5),
                        parallel=ParallelConfig(tp=8, zero_stage=0), seq_len=8192, micro_batch=8)
    llama8b_fp8 = RunConfig.from_dict(dict(llama8b.to_dict(), precision="fp8"))
    # the benchmark's headline layout: tensor parallelism inside a pair of GPUs, ZeRO-3 over the rest of the node
    llama8b_fsdp_tp2 = RunConfig(model=ModelConfig("llama3-8b", 128256, 32, 4096, 32, 8, 128, 14336, rope_theta=5e5),
                                 parallel=ParallelConfig(tp=2, zero_stage=3), seq_len=8192, micro_batch=2)
    moe = RunConfig(model=ModelConfig("moe-8x2b", 32000, 16, 2048, 16, 4, 128, 5632, n_experts=8, top_k=2),
                    parallel=ParallelConfig(ep=8, zero_stage=0), seq_len=4096, micro_batch=2)
    hybrid = RunConfig(model=ModelConfig("llama-3b-long", 32000, 28, 3072, 24, 8, 128, 8192),
                       parallel=ParallelConfig(tp=2, cp=2, pp=2, zero_stage=0), seq_len=32768, micro_batch=1, micro_batches=8,
                       activation_checkpointing=True)
    return {"gpt-cpu": gpt, "llama-1.1b-fsdp": llama1b, "llama3-8b-tp8": llama8b, "llama3-8b-tp8-fp8": llama8b_fp8,
            "llama3-8b-fsdp-tp2": llama8b_fsdp_tp2,
            "moe-8x2b-ep8": moe, "llama-3b-long-hybrid": hybrid}


PRESETS = _presets()


def load(source: str, env=None) -> RunConfig:
    """A preset name or the path of a JSON file; environment overrides are applied on top."""
    if source in PRESETS:
        cfg = RunConfig.from_dict(PRESETS[source].to_dict())
    else:
        with open(source) as f:
            cfg = RunConfig.from_dict(json.load(f))
    return apply_env(cfg, env)


__all__ = ["ModelConfig", "ParallelConfig", "OptimConfig", "RunConfig", "PRESETS", "load", "apply_env"]
