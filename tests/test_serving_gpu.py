"""KV-cache serving on the GPU: the native continuous-batching scheduler drives `LlamaKVModel` (chunked prefill into
the paged cache, batched decode on the split-K paged attention kernel); every generated token must be a (near-)argmax
of the logits that a full recomputation of its context gives, and the logits of the two paths must agree."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _setup(max_batched_tokens=96, kv_dtype=torch.bfloat16):
    from litetorch_b200.models.llama import LlamaConfig, LlamaEngine
    from litetorch_b200.models.llama_serving import LlamaKVModel
    from litetorch_b200.serving import ServingScheduler
    cfg = LlamaConfig.tiny()
    eng = LlamaEngine(cfg, "cuda", seed=4)
    model = LlamaKVModel(eng, num_blocks=256, block_size=16, kv_dtype=kv_dtype)
    sched = ServingScheduler(num_blocks=256, block_size=16, max_num_seqs=8, max_num_batched_tokens=max_batched_tokens, eos_id=-1)
    return cfg, eng, model, sched


def test_eight_requests_match_full_recompute():
    from litetorch_b200.serving import Request
    from litetorch_b200.ops import kernels as K
    cfg, eng, model, sched = _setup()
    g = torch.Generator().manual_seed(0)
    lens = [5, 17, 33, 64, 70, 100, 129, 150]          # prompts longer than the 96-token budget are prefilled in chunks
    reqs = [Request(i, torch.randint(3, cfg.vocab_size, (n,), generator=g).tolist(), max_new_tokens=6 + i) for i, n in enumerate(lens)]
    for r in reqs:
        sched.add_request(r)
    finished, steps = [], 0
    while len(finished) < len(reqs) and steps < 400:
        finished += sched.step(model)
        steps += 1
    assert len(finished) == len(reqs)
    assert sched.free_blocks == 256                     # every block went back to the pool
    worst = 0.0
    for r in reqs:
        assert len(r.generated_tokens) == r.max_new_tokens
        ctx = list(r.prompt_tokens)
        for t in r.generated_tokens:
            logits = eng.forward_logits(torch.tensor([ctx], device="cuda"))[0, -1].float()
            worst = max(worst, float(logits.max() - logits[t]))
            ctx.append(t)
    assert worst < 0.06, worst                          # the chosen token is the argmax up to bf16 noise of the two paths
    assert K.status_fetch() == 0


def test_decode_logits_equal_recompute_logits():
    cfg, eng, model, _ = _setup()
    g = torch.Generator().manual_seed(1)
    prompt = torch.randint(3, cfg.vocab_size, (90,), generator=g).tolist()
    blocks = list(range(10, 20))
    model.prefill_chunk(prompt[:48], 0, blocks, False)              # two chunks: the second reads the first from the cache
    model.prefill_chunk(prompt[48:], 48, blocks, True)
    ref = eng.forward_logits(torch.tensor([prompt], device="cuda"))[0, -1].float()
    err = float((model.last_logits[0].float() - ref).abs().max())
    assert err < 0.05, err
    nxt = int(ref.argmax())
    model.decode_batch([nxt], [len(prompt)], [blocks])
    ref2 = eng.forward_logits(torch.tensor([prompt + [nxt]], device="cuda"))[0, -1].float()
    err2 = float((model.last_logits[0].float() - ref2).abs().max())
    assert err2 < 0.05, err2


def test_ops_flash_decoding_and_moe_gate_use_the_kernels():
    import litetorch_b200 as lt
    from litetorch_b200.core import Tensor, _unwrap
    g = torch.Generator(device="cuda").manual_seed(0)
    q = torch.randn(3, 8, 1, 64, device="cuda", generator=g).bfloat16()
    k = torch.randn(3, 2, 700, 64, device="cuda", generator=g).bfloat16()
    v = torch.randn(3, 2, 700, 64, device="cuda", generator=g).bfloat16()
    o = _unwrap(lt.Ops.flash_decoding(Tensor(q), Tensor(k), Tensor(v), 4)).float()
    kk, vv = k.float().repeat_interleave(4, 1), v.float().repeat_interleave(4, 1)
    ref = torch.softmax(q.float() @ kk.transpose(-1, -2) / 8.0, -1) @ vv
    assert float((o - ref).abs().max()) < 2e-2
    x = torch.randn(64, 32, device="cuda", generator=g)
    wg = torch.randn(8, 32, device="cuda", generator=g)
    p, idx = lt.Ops.moe_gate(Tensor(x), Tensor(wg), 2)
    probs = torch.softmax(x @ wg.t(), -1)
    tp_, ti = probs.topk(2, -1)
    assert torch.equal(_unwrap(idx).long(), ti)
    assert float((_unwrap(p) - tp_ / tp_.sum(-1, keepdim=True)).abs().max()) < 1e-5
