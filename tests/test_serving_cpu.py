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


def test_prefix_reuse_copies_cached_blocks_and_gives_the_same_tokens():
    """With `prefix_cache_bytes` the K / V of a finished prompt's whole blocks are kept; a later prompt that starts with the
    same tokens gets them by a copy (fewer prompt tokens computed) and generates exactly what it generates without the
    cache; the snapshots respect their byte limit."""
    from litetorch_b200.models.llama import LlamaConfig, LlamaEngine, LocalWeights
    from litetorch_b200.models.llama_serving import LlamaKVModel
    from litetorch_b200.serving import Request, ServingScheduler
    cfg = LlamaConfig.tiny()
    eng = LlamaEngine(cfg, "cpu", weights=LocalWeights(cfg, "cpu", seed=4, param_dtype=torch.float32))
    g = torch.Generator().manual_seed(1)
    system = torch.randint(3, cfg.vocab_size, (45,), generator=g).tolist()          # a shared "system prompt"
    tails = [torch.randint(3, cfg.vocab_size, (n,), generator=g).tolist() for n in (7, 12, 3, 20)]
    prompts = [system + t for t in tails] + [system[:20] + tails[0]]                 # the last shares two blocks only

    def serve(cache_bytes, budget):
        model = LlamaKVModel(eng, num_blocks=64, block_size=8, kv_dtype=torch.float32, prefix_cache_bytes=cache_bytes)
        outs = []
        for i, p in enumerate(prompts):                                              # one after the other: later ones can reuse
            sched = ServingScheduler(num_blocks=64, block_size=8, max_num_seqs=2, max_num_batched_tokens=budget, eos_id=-1)
            r = Request(i, p, max_new_tokens=4)
            sched.add_request(r)
            while not sched.step(model):
                pass
            outs.append(list(r.generated_tokens))
        return outs, model

    plain, m0 = serve(0, 64)
    for budget in (64, 16, 11):                                                      # whole prompts, and chunks that split blocks
        cached, m1 = serve(1 << 20, budget)
        assert cached == plain
        # prefixes are findable at their full length and at power-of-two numbers of blocks: 32 of the 45 shared tokens
        # three times, 16 of 20 once
        if budget == 64:
            assert m1.prefill_tokens_reused == 3 * 32 + 16
        assert m1.prefill_tokens_reused >= 60                                        # chunk ends limit what a lookup can match
        assert m1.prefill_tokens_computed + m1.prefill_tokens_reused == m0.prefill_tokens_computed
    tiny, m2 = serve(2 * 5 * cfg.n_layers * cfg.n_kv_heads * 8 * cfg.head_dim * 4 + 1, 64)   # room for one five-block snapshot
    assert tiny == plain and len(m2._snap) == 1 and m2._snap_bytes <= m2.prefix_cache_bytes
