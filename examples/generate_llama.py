"""Text generation from a Hugging Face Llama directory (config.json + *.safetensors) on the serving path of this package:
weights converted by `models.llama_io`, continuous batching over a paged KV cache, CUDA-graph decode steps.

    python examples/generate_llama.py --model /models/llama --sentencepiece /models/llama/tokenizer.model \
        --prompt "The capital of France is" --prompt "Once upon a time" --max-new-tokens 64 --temperature 0.8 --top-p 0.95
    python examples/generate_llama.py --model export_dir --bytes --prompt "abc" --device cpu      # byte-level ids

Without a tokenizer (`--ids`), prompts are comma-separated token ids and the output is printed as ids.
"""
import argparse
import json
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch

from litetorch_b200.models import llama_io
from litetorch_b200.models.llama_serving import generate


def main(argv=None) -> dict:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", required=True, help="directory with config.json and *.safetensors")
    ap.add_argument("--prompt", action="append", required=True)
    ap.add_argument("--sentencepiece", default="")
    ap.add_argument("--bytes", action="store_true", help="byte-level ids (examples/prepare_data.py without a tokenizer)")
    ap.add_argument("--ids", action="store_true", help="prompts are comma-separated token ids")
    ap.add_argument("--max-new-tokens", type=int, default=32)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--top-k", type=int, default=0)
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--eos-id", type=int, default=-1)
    ap.add_argument("--device", default="cuda")
    args = ap.parse_args(argv)
    if args.sentencepiece:
        import sentencepiece as spm
        sp = spm.SentencePieceProcessor(model_file=args.sentencepiece)
        encode, decode = (lambda s: [sp.bos_id()] * (sp.bos_id() >= 0) + sp.encode(s)), sp.decode
        eos = sp.eos_id() if args.eos_id < 0 else args.eos_id
    elif args.bytes:
        encode = lambda s: list(s.encode("utf-8"))
        decode = lambda ids: bytes(i for i in ids if i < 256).decode("utf-8", errors="replace")
        eos = 256 if args.eos_id < 0 else args.eos_id
    else:
        encode = lambda s: [int(t) for t in s.split(",")]
        decode = lambda ids: ",".join(str(i) for i in ids)
        eos = args.eos_id
    kw = {}
    if args.device == "cpu":
        from litetorch_b200.models.llama import LocalWeights
        with open(os.path.join(args.model, "config.json")) as f:
            cfg = llama_io.config_from_hf(json.load(f))
        kw["weights"] = LocalWeights(cfg, "cpu", seed=0, param_dtype=torch.float32)
    engine = llama_io.load_pretrained(args.model, device=args.device, **kw)
    prompts = [encode(p) for p in args.prompt]
    t0 = time.time()
    outs = generate(engine, prompts, args.max_new_tokens, temperature=args.temperature, top_k=args.top_k, top_p=args.top_p,
                    seed=args.seed, eos_id=eos)
    dt = time.time() - t0
    texts = [decode(o) for o in outs]
    for p, t in zip(args.prompt, texts):
        print("%s -> %s" % (p, t))
    res = {"outputs": outs, "texts": texts, "seconds": round(dt, 3), "new_tokens": sum(len(o) for o in outs)}
    print("RESULT " + json.dumps(res))
    return res


if __name__ == "__main__":
    main()
