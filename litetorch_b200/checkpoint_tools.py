"""Offline work on `Trainer.save` checkpoints, without GPUs and without a process group:

    python -m litetorch_b200.checkpoint_tools info      --src /data/run1
    python -m litetorch_b200.checkpoint_tools reshard   --src /data/run1 --dst /data/run1_4gpu --world 4 --tp 2
    python -m litetorch_b200.checkpoint_tools export-hf --src /data/run1 --out /models/run1_hf [--dtype bfloat16]

A trainer checkpoint holds, per rank, the flat fp32 buffers of its weight provider (masters and AdamW moments).  The
three providers lay them out differently - everything on one rank (`LocalWeights`), rows of every matrix dealt to the
ranks (`ShardedWeights`, ZeRO-3), tensor-parallel slices whose rows are dealt to the data-parallel ranks
(`HybridWeights`) - but every layout is a function of the model, the world size and the tensor-parallel width alone,
so the whole state can be put together from the files and cut again for another layout.  `reshard` does that (a job
that was checkpointed on 8 GPUs continues on 4, or on one for debugging); `export-hf` writes the weights as a Hugging
Face directory.  The data loader's position is per rank and tied to the number of data-parallel replicas; it is not
carried over by `reshard`.  The reference has no counterpart.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import shutil
from typing import Dict, List, Tuple

import torch

from .models.llama import LlamaConfig, ParamSpec, param_specs
from .serialization import CheckpointError, read_tensors, save_sharded

QUANTITIES = ("master", "m", "v")


def _pad128(n: int) -> int:
    return (n + 127) // 128 * 128


def _slicer(cfg: LlamaConfig, tp: int):
    from .parallel.hybrid import TPSlicer
    return TPSlicer(cfg, tp)


class Layout:
    """Where every parameter lives in the flat buffers of one rank, for one provider / world size / tp."""

    def __init__(self, kind: str, cfg: LlamaConfig, world: int, tp: int):
        if kind not in ("LocalWeights", "ShardedWeights", "HybridWeights"):
            raise CheckpointError("unknown weight provider %r" % kind)
        if kind == "LocalWeights" and (world != 1 or tp != 1):
            raise CheckpointError("LocalWeights is a single-rank layout")
        if kind == "ShardedWeights" and tp != 1:
            raise CheckpointError("ShardedWeights has no tensor parallelism")
        if world % tp:
            raise CheckpointError("world size %d is not a multiple of tp %d" % (world, tp))
        self.kind, self.cfg, self.world, self.tp, self.dp = kind, cfg, world, tp, world // tp
        self.specs = param_specs(cfg)
        self.matrices = [s for s in self.specs if s.kind == "matrix"]
        self.vectors = [s for s in self.specs if s.kind == "vector"]
        self.slicer = _slicer(cfg, tp)
        self.n_matrix = max(s.offset + _pad128(math.prod(s.shape)) for s in self.matrices)
        self.n_vector = max(s.offset + _pad128(math.prod(s.shape)) for s in self.vectors)
        self.shard_off: Dict[str, int] = {}
        off = 0
        for s in self.matrices:
            rows, cols = self.slicer.local_shape(s)
            if rows % self.dp:
                raise CheckpointError("%s: %d rows do not divide over %d data-parallel ranks" % (s.name, rows, self.dp))
            self.shard_off[s.name] = off
            off += _pad128((rows // self.dp) * cols)
        self.n_shard = off

    @property
    def names(self) -> List[str]:
        return list(QUANTITIES) if self.kind == "LocalWeights" else ["master", "m", "v", "vec_master", "vec_m", "vec_v"]

    def _vec_name(self, q: str) -> str:
        return "vec_" + q

    # ---- one rank's buffers -> pieces of the full tensors
    def scatter_into(self, full: Dict[str, Dict[str, torch.Tensor]], rank: int, bufs: Dict[str, torch.Tensor]) -> None:
        dp_rank, tp_rank = divmod(rank, self.tp)
        for q in QUANTITIES:
            flat = bufs[q]
            for s in self.specs:
                dst = full[q][s.name]
                n = math.prod(s.shape)
                if self.kind == "LocalWeights":
                    base = s.offset if s.kind == "matrix" else self.n_matrix + s.offset
                    dst.copy_(flat[base:base + n].view(*s.shape))
                elif s.kind == "vector":
                    if rank == 0:                                   # replicated: one copy is enough
                        dst.copy_(bufs[self._vec_name(q)][s.offset:s.offset + n].view(*s.shape))
                else:
                    rows, cols = self.slicer.local_shape(s)
                    rpr = rows // self.dp
                    so = self.shard_off[s.name]
                    part = flat[so:so + rpr * cols].view(rpr, cols)
                    if self.tp == 1:
                        dst[dp_rank * rpr:(dp_rank + 1) * rpr].copy_(part)
                    else:
                        idx = self.slicer.row_index(s, tp_rank)
                        if idx is not None:                         # cut by rows: this rank's rows of the slice
                            dst.index_copy_(0, idx[dp_rank * rpr:(dp_rank + 1) * rpr], part)
                        else:                                       # cut by columns
                            c = s.shape[1] // self.tp
                            dst[dp_rank * rpr:(dp_rank + 1) * rpr, tp_rank * c:(tp_rank + 1) * c] = part

    # ---- full tensors -> one rank's buffers
    def gather_from(self, full: Dict[str, Dict[str, torch.Tensor]], rank: int) -> Dict[str, torch.Tensor]:
        dp_rank, tp_rank = divmod(rank, self.tp)
        out: Dict[str, torch.Tensor] = {}
        for q in QUANTITIES:
            if self.kind == "LocalWeights":
                flat = torch.zeros(self.n_matrix + self.n_vector, dtype=torch.float32)
            else:
                flat = torch.zeros(self.n_shard, dtype=torch.float32)
                vec = torch.zeros(self.n_vector, dtype=torch.float32)
            for s in self.specs:
                src = full[q][s.name]
                n = math.prod(s.shape)
                if self.kind == "LocalWeights":
                    base = s.offset if s.kind == "matrix" else self.n_matrix + s.offset
                    flat[base:base + n] = src.reshape(-1)
                elif s.kind == "vector":
                    vec[s.offset:s.offset + n] = src.reshape(-1)
                else:
                    part = self.slicer.take(s, src, tp_rank)
                    rpr = part.shape[0] // self.dp
                    mine = part[dp_rank * rpr:(dp_rank + 1) * rpr].reshape(-1)
                    so = self.shard_off[s.name]
                    flat[so:so + mine.numel()] = mine
            out[q] = flat
            if self.kind != "LocalWeights":
                out[self._vec_name(q)] = vec
        return out


def _resolve(directory: str) -> str:
    from .trainer import Trainer
    d = Trainer.latest_checkpoint(directory)
    if d is None:
        raise CheckpointError("no finished checkpoint in %s" % directory)
    return d


def read_manifest(directory: str) -> dict:
    with open(os.path.join(_resolve(directory), "trainer.manifest.json")) as f:
        return json.load(f)


def read_full_state(directory: str) -> Tuple[LlamaConfig, dict, Dict[str, Dict[str, torch.Tensor]]]:
    """(model configuration, manifest meta, {"master" | "m" | "v": {parameter name: whole fp32 tensor}}) of the newest
    finished checkpoint under `directory`."""
    d = _resolve(directory)
    man = read_manifest(directory)
    meta = man["meta"]
    cfg = LlamaConfig(**meta["model"])
    lay = Layout(meta["weights"], cfg, int(meta["world_size"]), int(meta["tp"]))
    if meta["names"] != lay.names:
        raise CheckpointError("the checkpoint holds %r, a %s layout has %r" % (meta["names"], lay.kind, lay.names))
    full = {q: {s.name: torch.zeros(*s.shape, dtype=torch.float32) for s in lay.specs} for q in QUANTITIES}
    for rank, fname in enumerate(man["files"]):
        tensors = read_tensors(os.path.join(d, fname))
        if len(tensors) != len(lay.names):
            raise CheckpointError("%s holds %d tensors, expected %d" % (fname, len(tensors), len(lay.names)))
        lay.scatter_into(full, rank, {n: t.reshape(-1) for n, t in zip(lay.names, tensors)})
    return cfg, meta, full


def write_state(directory: str, cfg: LlamaConfig, meta: dict, full: Dict[str, Dict[str, torch.Tensor]], world: int, tp: int,
                weights: str = "") -> str:
    """Write `full` as a finished trainer checkpoint for `world` ranks with tensor-parallel width `tp`; returns its path."""
    kind = weights or ("LocalWeights" if world == 1 else ("HybridWeights" if tp > 1 else "ShardedWeights"))
    lay = Layout(kind, cfg, world, tp)
    name = "step-%08d" % int(meta["step_count"])
    tmp, final = os.path.join(directory, "." + name + ".tmp"), os.path.join(directory, name)
    new_meta = dict(meta, weights=kind, world_size=world, tp=tp, names=lay.names)
    if os.path.isdir(tmp):
        shutil.rmtree(tmp)
    for rank in reversed(range(world)):                             # rank 0 last: it writes the manifest
        bufs = lay.gather_from(full, rank)
        save_sharded(tmp, [bufs[n] for n in lay.names], rank, world, tag="trainer", meta=new_meta)
    if os.path.isdir(final):
        shutil.rmtree(final)
    os.replace(tmp, final)
    with open(os.path.join(directory, "LATEST.tmp"), "w") as f:
        f.write(name)
    os.replace(os.path.join(directory, "LATEST.tmp"), os.path.join(directory, "LATEST"))
    return final


def reshard(src: str, dst: str, world: int, tp: int = 1, weights: str = "") -> str:
    cfg, meta, full = read_full_state(src)
    os.makedirs(dst, exist_ok=True)
    return write_state(dst, cfg, meta, full, world, tp, weights)


def export_hf(src: str, out: str, dtype=torch.bfloat16) -> None:
    """The master weights of a checkpoint as `config.json` + `model.safetensors` for `transformers`."""
    from safetensors.torch import save_file
    from .models import llama_io
    cfg, _, full = read_full_state(src)
    sd = llama_io.to_hf(cfg, [full["master"][s.name] for s in param_specs(cfg)])
    os.makedirs(out, exist_ok=True)
    save_file({k: v.to(dtype).contiguous() for k, v in sd.items()}, os.path.join(out, "model.safetensors"), metadata={"format": "pt"})
    hf_cfg = llama_io.config_to_hf(cfg)
    hf_cfg["torch_dtype"] = str(dtype).replace("torch.", "")
    with open(os.path.join(out, "config.json"), "w") as f:
        json.dump(hf_cfg, f, indent=1)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    sub = ap.add_subparsers(dest="cmd", required=True)
    a = sub.add_parser("info")
    a.add_argument("--src", required=True)
    a = sub.add_parser("reshard")
    a.add_argument("--src", required=True)
    a.add_argument("--dst", required=True)
    a.add_argument("--world", type=int, required=True)
    a.add_argument("--tp", type=int, default=1)
    a.add_argument("--weights", default="", choices=["", "LocalWeights", "ShardedWeights", "HybridWeights"])
    a = sub.add_parser("export-hf")
    a.add_argument("--src", required=True)
    a.add_argument("--out", required=True)
    a.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float16", "float32"])
    args = ap.parse_args(argv)
    if args.cmd == "info":
        meta = read_manifest(args.src)["meta"]
        cfg = LlamaConfig(**meta["model"])
        print(json.dumps({"checkpoint": _resolve(args.src), "step_count": meta["step_count"], "weights": meta["weights"],
                          "world_size": meta["world_size"], "tp": meta["tp"], "model": meta["model"]["name"],
                          "parameters": cfg.num_params()}, indent=1))
    elif args.cmd == "reshard":
        print(reshard(args.src, args.dst, args.world, args.tp, args.weights))
    else:
        export_hf(args.src, args.out, getattr(torch, args.dtype))
        print(args.out)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
