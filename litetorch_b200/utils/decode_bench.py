"""Decode throughput of the KV-cache serving path (`models.llama_serving.LlamaKVModel.decode_batch`).

    python -m litetorch_b200.utils.decode_bench [--model llama-1.1b] [--batches 1,32,128] [--contexts 2048,16384]

For every (batch, context) pair the paged cache is filled with random keys / values for `context` positions per
sequence and one decode step is timed (CUDA events, 10 timed steps after 3 warm-up steps; the step's working set -
the weights plus the batch's KV blocks - is larger than the L2 except for batch 1 at 2 k, where the weights alone
are).  A decode step must read every weight once and every cached K / V byte of the batch once, so the roofline is
(weight bytes + KV bytes) / measured copy bandwidth; the table reports tokens/s and the achieved fraction.
One JSON line per pair, then a summary line.
"""
from __future__ import annotations

import argparse
import json

import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama-1.1b", choices=["llama-1.1b", "llama-tiny", "llama3-8b"])
    ap.add_argument("--batches", default="1,32,128")
    ap.add_argument("--contexts", default="2048,16384")
    ap.add_argument("--no-graphs", action="store_true", help="launch every kernel of a step instead of replaying a CUDA graph")
    ap.add_argument("--hbm-gbs", type=float, default=6552.0, help="measured copy bandwidth used as the roofline denominator")
    a = ap.parse_args()
    from ..models.llama import LlamaConfig, LlamaEngine
    from ..models.llama_serving import LlamaKVModel
    from ..ops import kernels as K
    cfg = {"llama-1.1b": LlamaConfig.llama_1b, "llama-tiny": LlamaConfig.tiny, "llama3-8b": LlamaConfig.llama3_8b}[a.model]()
    batches = [int(x) for x in a.batches.split(",")]
    contexts = [int(x) for x in a.contexts.split(",")]
    import dataclasses
    cfg = dataclasses.replace(cfg, max_seq=max(contexts) + 64)
    dev = torch.device("cuda")
    # inference only: the bf16 parameters alone (no gradients, no optimizer state)
    eng = LlamaEngine.__new__(LlamaEngine)
    from ..models.llama import LocalWeights, kernels_for, rope_tables

    class _InferenceWeights(LocalWeights):
        def __init__(self, cfg, device, seed):
            from ..models.llama import param_specs
            import math
            self.cfg, self.K = cfg, kernels_for(device)
            self.specs = param_specs(cfg)
            self.by_name = {s.name: s for s in self.specs}
            sizes = {"matrix": 0, "vector": 0}
            for s in self.specs:
                sizes[s.kind] = max(sizes[s.kind], s.offset + (math.prod(s.shape) + 127) // 128 * 128)
            self.n_matrix, self.n_vector = sizes["matrix"], sizes["vector"]
            self.flat_p = torch.empty(self.n_matrix + self.n_vector, dtype=torch.bfloat16, device=device)
            self.flat_p[:self.n_matrix].normal_(0.0, cfg.init_std, generator=torch.Generator(device=device).manual_seed(seed))
            self.flat_p[self.n_matrix:].fill_(1.0)

    eng.cfg, eng.device, eng.K = cfg, dev, kernels_for(dev)
    eng.w = _InferenceWeights(cfg, dev, 0)
    eng.cos, eng.sin = rope_tables(cfg, dev)
    weight_bytes = eng.w.n_matrix * 2 - cfg.vocab_size * cfg.d_model * 2          # the embedding table is only gathered from
    bs = 16
    rows = []
    for B in batches:
        for ctx in contexts:
            blocks_per_seq = (ctx + 1 + bs - 1) // bs
            model = LlamaKVModel(eng, num_blocks=B * blocks_per_seq + 1, block_size=bs, graphs=not a.no_graphs)
            for layer in range(cfg.n_layers):
                model.cache.k[layer].normal_(0.0, 1.0)
                model.cache.v[layer].normal_(0.0, 1.0)
            tables = [list(range(1 + s * blocks_per_seq, 1 + (s + 1) * blocks_per_seq)) for s in range(B)]
            toks, pos = [1] * B, [ctx] * B
            for _ in range(3):
                model.decode_batch(toks, pos, tables)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            n0 = K.launch_count()
            e0.record()
            for _ in range(10):
                model.decode_batch(toks, pos, tables)
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / 10
            kv_bytes = B * (ctx + 1) * model.kv_bytes_per_token
            floor_ms = (weight_bytes + kv_bytes) / (a.hbm_gbs * 1e9) * 1e3
            row = {"model": cfg.name, "batch": B, "context": ctx, "ms_per_step": round(ms, 3), "tokens_per_s": round(B / ms * 1e3, 1),
                   "weight_gb": round(weight_bytes / 1e9, 2), "kv_gb": round(kv_bytes / 1e9, 2), "roofline_ms": round(floor_ms, 3),
                   "fraction_of_measured_hbm_roofline": round(floor_ms / ms, 3), "launches_per_step": (K.launch_count() - n0) // 10}
            print(json.dumps(row), flush=True)
            rows.append(row)
            del model
            torch.cuda.empty_cache()
    print(json.dumps({"summary": [(r["batch"], r["context"], r["tokens_per_s"], r["fraction_of_measured_hbm_roofline"]) for r in rows],
                      "device_status": K.status_fetch()}))


if __name__ == "__main__":
    main()
