"""The KV-cache serving path on the CPU twin of the kernels: scheduler + chunked prefill + paged decode give exactly the
tokens of greedy decoding by full recomputation (fp32, so the argmax is unambiguous)."""
import torch


def test_kv_cache_serving_matches_full_recompute_cpu():
    from litetorch_b200.models.llama import LlamaConfig, LlamaEngine, LocalWeights
    from litetorch_b200.models.llama_serving import LlamaKVModel
    from litetorch_b200.serving import Request, ServingScheduler
    cfg = LlamaConfig.tiny()
    eng = LlamaEngine(cfg, "cpu", weights=LocalWeights(cfg, "cpu", seed=4, param_dtype=torch.float32))
    model = LlamaKVModel(eng, num_blocks=64, block_size=8, kv_dtype=torch.float32)
    sched = ServingScheduler(num_blocks=64, block_size=8, max_num_seqs=4, max_num_batched_tokens=24, eos_id=-1)
    g = torch.Generator().manual_seed(0)
    reqs = [Request(i, torch.randint(3, cfg.vocab_size, (n,), generator=g).tolist(), max_new_tokens=3 + i)
            for i, n in enumerate([5, 17, 40, 9, 30])]
    for r in reqs:
        sched.add_request(r)
    done, steps = [], 0
    while len(done) < len(reqs) and steps < 200:
        done += sched.step(model)
        steps += 1
    assert len(done) == len(reqs) and sched.free_blocks == 64
    for r in reqs:
        ctx = list(r.prompt_tokens)
        for t in r.generated_tokens:
            logits = eng.forward_logits(torch.tensor([ctx]))[0, -1]
            assert int(logits.argmax()) == t
            ctx.append(t)
        assert len(r.generated_tokens) == r.max_new_tokens
