"""Pre-training loop on a token file: configuration -> Trainer -> TokenStream -> warm-up + cosine schedule -> periodic
evaluation and crash-consistent checkpoints -> resume.  One process per GPU:

    python examples/train_llama.py --data tokens.bin --config llama-1.1b-fsdp --steps 1000 --ckpt /data/run1
    python -m torch.distributed.run --nproc-per-node 8 examples/train_llama.py --data tokens.bin \
        --config llama3-8b-fsdp-tp2 --ckpt /data/run1
    python -m litetorch_b200.parallel.elastic --nproc 8 --max-restarts 3 examples/train_llama.py --data tokens.bin ...

`--data` is a flat file of uint16 (or `--dtype uint32`) token ids; `--tiny --device cpu` runs a toy model on the CPU
(what the tests do).  Started again with the same `--ckpt`, the job continues from the newest finished checkpoint with
the batches it would have seen: the loader's position is part of the checkpoint.  Under the elastic launcher the
process also beats in the launcher's store, so a hung rank is noticed and the group is restarted.
"""
import argparse
import json
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch

import litetorch_b200 as lt
from litetorch_b200.models.llama import LlamaConfig
from litetorch_b200.parallel import elastic
from litetorch_b200.trainer import Trainer


def main(argv=None) -> dict:
    ap = argparse.ArgumentParser()
    ap.add_argument("--data", required=True, help="flat binary file of token ids")
    ap.add_argument("--dtype", default="uint16", choices=["uint16", "uint32"])
    ap.add_argument("--config", default="llama-1.1b-fsdp", help="a preset name or a JSON job description")
    ap.add_argument("--tiny", action="store_true", help="a two-layer toy model instead of the configuration's")
    ap.add_argument("--device", default=None, help="default: cuda:<LOCAL_RANK>")
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--seq-len", type=int, default=0, help="default: the configuration's")
    ap.add_argument("--batch", type=int, default=0, help="sequences per rank and step (default: the configuration's)")
    ap.add_argument("--micro-batches", type=int, default=1)
    ap.add_argument("--lr", type=float, default=0.0, help="peak learning rate (default: the configuration's)")
    ap.add_argument("--warmup", type=int, default=10, help="steps of linear warm-up before the cosine decay")
    ap.add_argument("--min-lr-ratio", type=float, default=0.1)
    ap.add_argument("--grad-clip", type=float, default=0.0, help="unsharded weights only")
    ap.add_argument("--eval-every", type=int, default=0)
    ap.add_argument("--ckpt", default="", help="checkpoint directory (resumed from when it holds a checkpoint)")
    ap.add_argument("--ckpt-every", type=int, default=50)
    ap.add_argument("--metrics", default="", help="JSON-lines file for per-step metrics")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--init-hf", default="", help="start from a Hugging Face Llama directory (fine-tuning): its config.json "
                    "replaces the configuration's model, its weights are loaded unless --ckpt already holds a checkpoint")
    ap.add_argument("--export-hf", default="", help="write the final weights as a Hugging Face directory")
    args = ap.parse_args(argv)

    elastic.start_heartbeat()                               # a no-op unless the elastic launcher started this process
    run = lt.config.load(args.config)
    cfg = LlamaConfig.tiny() if args.tiny else run.llama_config()
    if args.init_hf:
        from litetorch_b200.models import llama_io
        with open(os.path.join(args.init_hf, "config.json")) as f:
            cfg = llama_io.config_from_hf(json.load(f))
    seq_len = args.seq_len or min(run.seq_len, cfg.max_seq)
    batch = args.batch or run.micro_batch
    peak = args.lr or run.optim.lr
    world = int(os.environ.get("WORLD_SIZE", "1"))
    kw = dict(lr=peak, betas=(run.optim.beta1, run.optim.beta2), eps=run.optim.eps, weight_decay=run.optim.weight_decay,
              seed=args.seed, activation_checkpointing=run.activation_checkpointing, micro_batches=args.micro_batches,
              grad_clip=args.grad_clip)
    if args.device:
        kw.update(device=args.device)
        if args.device == "cpu":
            kw.update(param_dtype=torch.float32)
    if world == 1:
        kw.update(parallel="none")
    else:
        kw.update(tp=run.parallel.tp, parallel="hybrid" if run.parallel.tp > 1 else "auto")
    trainer = Trainer(cfg, **kw)
    from litetorch_b200.utils.logging import get_logger
    log = get_logger("train")
    say = log.info

    # every data-parallel replica reads its own windows; the ranks of a tensor-parallel group read the same ones
    stream = lt.data.TokenStream(args.data, seq_len, batch, dtype=args.dtype, shuffle=True, seed=args.seed,
                                 rank=trainer.dp_rank, world=max(trainer.dp, 1))
    held_out = lt.data.TokenStream(args.data, seq_len, batch, dtype=args.dtype, shuffle=True, seed=args.seed + 1,
                                   rank=trainer.dp_rank, world=max(trainer.dp, 1)) if args.eval_every else None
    if args.metrics:
        trainer.log_metrics(args.metrics)
    if args.init_hf and not (args.ckpt and Trainer.latest_checkpoint(args.ckpt)):
        llama_io.load_into(trainer.engine, llama_io.read_state_dict(args.init_hf))     # every rank keeps its part
        say("initialised from %s" % args.init_hf)
    if args.ckpt and Trainer.latest_checkpoint(args.ckpt):
        try:
            trainer.load(args.ckpt, loader=stream)
        except RuntimeError as e:
            # a checkpoint that was re-cut for another world size carries no loader position: the weights and the
            # optimizer resume, the data starts from the beginning of an epoch chosen by the step count
            if "loader" not in str(e) and "token stream" not in str(e):
                raise
            trainer.load(args.ckpt)
            stream.load_state_dict(dict(stream.state_dict(), epoch=trainer.engine.step_count // max(1, stream.batches_per_epoch) + 1,
                                        position=0))
            say("the checkpoint has no loader position for this layout: data restarts at epoch %d" % stream.epoch)
        say("resumed from %s at step %d" % (Trainer.latest_checkpoint(args.ckpt), trainer.engine.step_count))

    # the rate depends on the step count alone: a resumed job continues on the same curve
    sched = lt.optim.WarmupCosineLR(trainer, args.warmup, args.steps, args.min_lr_ratio, last_epoch=trainer.engine.step_count)

    losses, evals = [], []
    batches = iter(stream)
    t0 = time.time()
    while trainer.engine.step_count < args.steps:
        tokens, targets = next(batches)
        losses.append(trainer.step(tokens, targets))
        sched.step()
        step = trainer.engine.step_count
        if args.eval_every and step % args.eval_every == 0:
            tk, tg = next(iter(held_out))
            evals.append((step, trainer.evaluate(tk, tg)))
            say("step %d  loss %.4f  eval %.4f  lr %.2e" % (step, losses[-1], evals[-1][1], trainer.get_lr()))
        if args.ckpt and (step % args.ckpt_every == 0 or step == args.steps):
            trainer.save(args.ckpt, keep=2, loader=stream, background=step != args.steps)
    trainer.finish_save()
    if args.export_hf:
        from litetorch_b200.models import llama_io
        llama_io.save_pretrained(trainer.engine, args.export_hf, dtype=torch.float32 if args.device == "cpu" else torch.bfloat16)
    out = {"steps": trainer.engine.step_count, "losses": losses, "evals": evals, "seconds": round(time.time() - t0, 3),
           "epoch": stream.epoch, "position": stream.position}
    if trainer.rank == 0:
        print("RESULT " + json.dumps(out), flush=True)
    return out


if __name__ == "__main__":
    main()
