"""examples/train_llama.py end to end on the CPU: a toy model learns a periodic token file, an interrupted run that is
started again with the same checkpoint directory ends on the curve of the uninterrupted one, and the same script runs
as two data-parallel gloo ranks."""
import json
import os
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SCRIPT = os.path.join(ROOT, "examples", "train_llama.py")


def _tokens(path, n=40000, period=37, vocab=512):
    rng = np.random.default_rng(0)
    base = rng.integers(3, vocab, size=period)
    np.tile(base, n // period + 1)[:n].astype(np.uint16).tofile(path)


def _run(args, nproc=1, port=29931, timeout=900):
    cmd = [sys.executable, SCRIPT] if nproc == 1 else [
        sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(nproc), "--master-addr", "127.0.0.1",
        "--master-port", str(port), SCRIPT]
    r = subprocess.run(cmd + args, capture_output=True, text=True, timeout=timeout, env=dict(os.environ, OMP_NUM_THREADS="2"))
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    return json.loads([l for l in r.stdout.splitlines() if l.startswith("RESULT ")][-1][7:])


def test_example_trains_evaluates_and_resumes_on_the_same_curve(tmp_path):
    data = str(tmp_path / "tokens.bin")
    _tokens(data)
    common = ["--data", data, "--tiny", "--device", "cpu", "--config", "llama-1.1b-fsdp", "--seq-len", "32", "--batch", "4",
              "--lr", "3e-3", "--warmup", "4", "--eval-every", "10", "--grad-clip", "1.0"]
    whole = _run(common + ["--steps", "30", "--ckpt", str(tmp_path / "a"), "--ckpt-every", "10",
                           "--metrics", str(tmp_path / "m.jsonl")])
    assert whole["steps"] == 30 and whole["losses"][-1] < 0.6 * whole["losses"][0]
    assert [s for s, _ in whole["evals"]] == [10, 20, 30] and whole["evals"][-1][1] < whole["evals"][0][1]
    assert len(open(tmp_path / "m.jsonl").read().splitlines()) == 30
    # an interrupted job: the same 30-step job whose newest finished checkpoint is the one of step 20
    part = _run(common + ["--steps", "30", "--ckpt", str(tmp_path / "c"), "--ckpt-every", "20"])
    assert part["losses"] == whole["losses"]                      # same seed, same data order: deterministic on the CPU
    os.remove(os.path.join(str(tmp_path / "c"), "LATEST"))        # forget the final checkpoint: step 20 is the newest left
    with open(os.path.join(str(tmp_path / "c"), "LATEST"), "w") as f:
        f.write("step-00000020")
    rest = _run(common + ["--steps", "30", "--ckpt", str(tmp_path / "c"), "--ckpt-every", "20"])
    assert rest["steps"] == 30 and len(rest["losses"]) == 10
    assert all(abs(a - b) < 1e-5 for a, b in zip(rest["losses"], whole["losses"][20:]))
    assert (rest["epoch"], rest["position"]) == (whole["epoch"], whole["position"])


def test_example_runs_as_two_data_parallel_ranks(tmp_path):
    data = str(tmp_path / "tokens.bin")
    _tokens(data)
    out = _run(["--data", data, "--tiny", "--device", "cpu", "--config", "llama-1.1b-fsdp", "--seq-len", "32", "--batch", "2",
                "--lr", "3e-3", "--warmup", "2", "--steps", "8", "--ckpt", str(tmp_path / "ck"), "--ckpt-every", "4",
                "--eval-every", "4"], nproc=2)
    assert out["steps"] == 8 and out["losses"][-1] < out["losses"][0]
    assert [s for s, _ in out["evals"]] == [4, 8] and out["evals"][1][1] < out["evals"][0][1]      # averaged over the two ranks
    assert sorted(os.listdir(tmp_path / "ck")) == ["LATEST", "step-00000004", "step-00000008"]
    assert "trainer.rank00001.ltw1" in os.listdir(tmp_path / "ck" / "step-00000008")


def test_prepare_data_then_train_then_export_then_generate(tmp_path):
    """The whole path a user walks: text -> token file -> a few training steps -> Hugging Face export -> generation."""
    import torch
    sys.path.insert(0, ROOT)
    from litetorch_b200.models import llama_io
    from litetorch_b200.models.llama import LlamaConfig, LlamaEngine, LocalWeights
    text = tmp_path / "corpus.txt"
    text.write_text(("the quick brown fox jumps over the lazy dog\n" * 40 + "\n") * 30)
    r = subprocess.run([sys.executable, os.path.join(ROOT, "examples", "prepare_data.py"), "--input", str(text), "--out",
                        str(tmp_path / "tokens.bin")], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    meta = json.loads(r.stdout.splitlines()[-1])
    assert meta["documents"] == 30 and meta["vocab_size"] == 257 and meta["tokens"] == 30 * (40 * 44 + 1)
    toks = np.fromfile(str(tmp_path / "tokens.bin"), dtype=np.uint16)
    assert len(toks) == meta["tokens"] and int(toks.max()) == 256 and bytes(toks[:9].astype(np.uint8)) == b"the quick"
    # a small byte-level model, trained a little in-process on that file
    import litetorch_b200 as lt
    cfg = LlamaConfig(vocab_size=264, n_layers=2, d_model=64, n_heads=4, n_kv_heads=2, head_dim=16, ffn=128, max_seq=128, name="bytes")
    engine = LlamaEngine(cfg, "cpu", weights=LocalWeights(cfg, "cpu", seed=0, param_dtype=torch.float32), lr=3e-3, weight_decay=0.0)
    stream = lt.data.TokenStream(str(tmp_path / "tokens.bin"), 64, 8, seed=0, rank=0, world=1)
    it = iter(stream)
    losses = [float(engine.train_step(*next(it))) for _ in range(60)]
    assert losses[-1] < 0.5 * losses[0]
    llama_io.save_pretrained(engine, str(tmp_path / "export"), dtype=torch.float32)
    g = subprocess.run([sys.executable, os.path.join(ROOT, "examples", "generate_llama.py"), "--model", str(tmp_path / "export"),
                        "--bytes", "--device", "cpu", "--prompt", "the quick brown fox jumps over the lazy dog\nthe quick ",
                        "--max-new-tokens", "10"], capture_output=True, text=True, timeout=600)
    assert g.returncode == 0, g.stdout[-2000:] + g.stderr[-3000:]
    res = json.loads([l for l in g.stdout.splitlines() if l.startswith("RESULT ")][-1][7:])
    assert res["new_tokens"] == 10 and len(res["texts"][0]) > 0


def test_example_continues_from_a_checkpoint_recut_for_fewer_ranks(tmp_path):
    """Two data-parallel ranks train and checkpoint; the checkpoint is re-cut for one rank and the same script goes on
    from its step count (weights and optimizer resume, the data position does not carry over)."""
    sys.path.insert(0, ROOT)
    from litetorch_b200 import checkpoint_tools
    data = str(tmp_path / "tokens.bin")
    _tokens(data)
    common = ["--data", data, "--tiny", "--device", "cpu", "--config", "llama-1.1b-fsdp", "--seq-len", "32", "--batch", "2",
              "--lr", "3e-3", "--warmup", "2", "--ckpt-every", "6"]
    two = _run(common + ["--steps", "6", "--ckpt", str(tmp_path / "ck2")], nproc=2, port=29951)
    assert two["steps"] == 6
    checkpoint_tools.reshard(str(tmp_path / "ck2"), str(tmp_path / "ck1"), world=1)
    one = _run(common + ["--steps", "12", "--ckpt", str(tmp_path / "ck1")])
    assert one["steps"] == 12 and len(one["losses"]) == 6 and one["losses"][0] < two["losses"][0]


def test_example_fine_tunes_from_a_hugging_face_directory_and_exports(tmp_path):
    import torch
    sys.path.insert(0, ROOT)
    from litetorch_b200.models import llama_io
    from litetorch_b200.models.llama import LlamaConfig, LlamaEngine, LocalWeights
    data = str(tmp_path / "tokens.bin")
    _tokens(data, vocab=256)
    cfg = LlamaConfig(vocab_size=256, n_layers=2, d_model=64, n_heads=4, n_kv_heads=2, head_dim=16, ffn=128, max_seq=64, name="base")
    base = LlamaEngine(cfg, "cpu", weights=LocalWeights(cfg, "cpu", seed=11, param_dtype=torch.float32))
    llama_io.save_pretrained(base, str(tmp_path / "base"), dtype=torch.float32)
    out = _run(["--data", data, "--device", "cpu", "--init-hf", str(tmp_path / "base"), "--seq-len", "32", "--batch", "4",
                "--lr", "2e-3", "--warmup", "2", "--steps", "12", "--export-hf", str(tmp_path / "tuned")])
    # the first loss is the base model's loss on the first batch: the weights came from the directory, not from a seed
    import litetorch_b200 as lt
    stream = lt.data.TokenStream(data, 32, 4, shuffle=True, seed=0, rank=0, world=1)
    tok, tgt = stream.next()
    assert abs(out["losses"][0] - float(base.eval_loss(tok, tgt))) < 1e-4 and out["losses"][-1] < out["losses"][0]
    tuned = llama_io.load_pretrained(str(tmp_path / "tuned"), device="cpu", weights=LocalWeights(cfg, "cpu", seed=0, param_dtype=torch.float32))
    assert float(tuned.eval_loss(tok, tgt)) < float(base.eval_loss(tok, tgt))
