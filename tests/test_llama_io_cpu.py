"""The Llama engine against `transformers`' own Llama: a randomly initialised Hugging Face model converted into the
engine gives the same logits and the same loss, the conversion back reproduces the state dict, and a directory written by
`save_pretrained` is loaded by `transformers` and by `load_pretrained`."""
import pytest
import torch

def _hf_model(seed=0, **kw):
    pytest.importorskip("transformers")            # imported by the tests that need it, not at collection time
    from transformers import LlamaConfig as HC, LlamaForCausalLM
    torch.manual_seed(seed)
    args = dict(vocab_size=384, hidden_size=128, intermediate_size=320, num_hidden_layers=2, num_attention_heads=4,
                num_key_value_heads=2, head_dim=32, max_position_embeddings=128, rms_norm_eps=1e-5, rope_theta=10000.0,
                tie_word_embeddings=False, attention_bias=False, mlp_bias=False)
    args.update(kw)
    hc = HC(**args)
    model = LlamaForCausalLM(hc).eval().float()
    with torch.no_grad():                     # norm gains away from 1 so that a swapped pair of norms would show
        for n, p in model.named_parameters():
            if "norm" in n:
                p.add_(torch.randn_like(p) * 0.1)
    return hc, model


def test_engine_reproduces_the_hugging_face_forward_pass_and_loss():
    from litetorch_b200.models import llama_io
    from litetorch_b200.models.llama import LlamaEngine, LocalWeights
    hc, model = _hf_model()
    cfg = llama_io.config_from_hf(hc)
    assert (cfg.n_heads, cfg.n_kv_heads, cfg.head_dim, cfg.ffn, cfg.n_layers) == (4, 2, 32, 320, 2)
    engine = LlamaEngine(cfg, "cpu", weights=LocalWeights(cfg, "cpu", seed=1, param_dtype=torch.float32))
    llama_io.load_into(engine, model.state_dict())
    tok = torch.randint(0, cfg.vocab_size, (2, 48), generator=torch.Generator().manual_seed(3))
    with torch.no_grad():
        ref = model(tok).logits
    got = engine.forward_logits(tok)
    assert float((got - ref).abs().max()) < 2e-4 * max(1.0, float(ref.abs().max()))
    tgt = torch.randint(0, cfg.vocab_size, (2, 48), generator=torch.Generator().manual_seed(4))
    loss_ref = torch.nn.functional.cross_entropy(ref.view(-1, cfg.vocab_size), tgt.view(-1))
    loss = engine.forward_backward(tok, tgt)
    assert abs(float(loss) - float(loss_ref)) < 1e-4
    # gradients too: the engine's flat gradient against autograd through the Hugging Face model
    model.zero_grad()
    torch.nn.functional.cross_entropy(model(tok).logits.view(-1, cfg.vocab_size), tgt.view(-1)).backward()
    hf_grads = llama_io.from_hf(cfg, {n: p.grad for n, p in model.named_parameters()})
    for s, g in zip(engine.w.specs, hf_grads):
        mine = engine.w.g(s.name).float()
        assert float((mine - g.view_as(mine)).abs().max()) < 1e-4 * max(1.0, float(g.abs().max())), s.name


def test_conversion_round_trip_and_tied_embeddings():
    from litetorch_b200.models import llama_io
    hc, model = _hf_model(seed=1)
    cfg = llama_io.config_from_hf(hc)
    sd = {k: v.clone() for k, v in model.state_dict().items()}
    back = llama_io.to_hf(cfg, llama_io.from_hf(cfg, sd))
    assert set(back) == set(sd)
    for k in sd:
        assert torch.equal(back[k], sd[k].float()), k
    tied = {k: v for k, v in sd.items() if k != "lm_head.weight"}
    tensors = llama_io.from_hf(cfg, tied)
    assert torch.equal(tensors[-1], sd["model.embed_tokens.weight"])
    with pytest.raises(ValueError):
        llama_io.config_from_hf(dict(llama_io.config_to_hf(cfg), attention_bias=True))
    with pytest.raises(ValueError):
        llama_io.from_hf(llama_io.config_from_hf(dict(llama_io.config_to_hf(cfg), intermediate_size=512)), sd)


def test_save_pretrained_is_read_by_transformers_and_by_load_pretrained(tmp_path):
    pytest.importorskip("safetensors")
    pytest.importorskip("transformers")
    from transformers import LlamaForCausalLM
    from litetorch_b200.models import llama_io
    from litetorch_b200.models.llama import LlamaConfig, LlamaEngine, LocalWeights
    cfg = LlamaConfig(vocab_size=256, n_layers=2, d_model=64, n_heads=4, n_kv_heads=2, head_dim=16, ffn=128, max_seq=64,
                      name="tiny")
    engine = LlamaEngine(cfg, "cpu", weights=LocalWeights(cfg, "cpu", seed=5, param_dtype=torch.float32))
    tok = torch.randint(0, cfg.vocab_size, (2, 33), generator=torch.Generator().manual_seed(6))
    engine.train_step(tok[:, :-1], tok[:, 1:])                    # weights that are not the initial ones
    out = str(tmp_path / "export")
    llama_io.save_pretrained(engine, out, dtype=torch.float32)
    hf = LlamaForCausalLM.from_pretrained(out, torch_dtype=torch.float32).eval()
    with torch.no_grad():
        ref = hf(tok[:, :-1]).logits
    assert float((engine.forward_logits(tok[:, :-1]) - ref).abs().max()) < 2e-4
    again = llama_io.load_pretrained(out, device="cpu", weights=LocalWeights(cfg, "cpu", seed=9, param_dtype=torch.float32))
    assert again.cfg.ffn == 128 and float((again.forward_logits(tok[:, :-1]) - ref).abs().max()) < 2e-4


def test_generate_equals_transformers_greedy_decoding_and_sampling_is_seeded():
    from litetorch_b200.models import llama_io
    from litetorch_b200.models.llama import LlamaEngine, LocalWeights
    from litetorch_b200.models.llama_serving import Sampler, generate
    hc, model = _hf_model(seed=2)
    cfg = llama_io.config_from_hf(hc)
    engine = LlamaEngine(cfg, "cpu", weights=LocalWeights(cfg, "cpu", seed=1, param_dtype=torch.float32))
    llama_io.load_into(engine, model.state_dict())
    g = torch.Generator().manual_seed(8)
    prompts = [torch.randint(3, cfg.vocab_size, (n,), generator=g).tolist() for n in (5, 19, 11)]
    ours = generate(engine, prompts, 8, block_size=4, max_num_batched_tokens=16)
    for p, o in zip(prompts, ours):
        with torch.no_grad():
            ref = model.generate(torch.tensor([p]), max_new_tokens=8, do_sample=False, pad_token_id=0, eos_token_id=None)
        assert ref[0, len(p):].tolist() == o
    shared = [prompts[1] + [7, 8, 9], prompts[1] + [11, 12]]                    # a common 19-token prefix
    assert generate(engine, shared, 4, block_size=4, max_num_seqs=1, prefix_cache_bytes=1 << 20) == generate(engine, shared, 4, block_size=4)
    # sampling: top_k = 1 is greedy, a seed reproduces a run, another seed changes it, tokens stay inside the top-k set
    assert generate(engine, prompts, 8, temperature=0.8, top_k=1) == ours
    a = generate(engine, prompts, 8, temperature=1.5, top_k=20, top_p=0.9, seed=5)
    assert a == generate(engine, prompts, 8, temperature=1.5, top_k=20, top_p=0.9, seed=5)
    assert a != generate(engine, prompts, 8, temperature=1.5, top_k=20, top_p=0.9, seed=6)
    logits = torch.randn(4, 50, generator=g)
    s = Sampler(temperature=1.0, top_k=3, top_p=1.0, seed=1)
    top3 = logits.topk(3, -1).indices
    for _ in range(20):
        t = s(logits)
        assert all(int(t[i]) in top3[i].tolist() for i in range(4))
    nucleus = Sampler(temperature=1.0, top_p=1e-6, seed=1)          # a vanishing nucleus keeps only the best token
    assert torch.equal(nucleus(logits), logits.argmax(-1))
    with pytest.raises(ValueError):
        generate(engine, [[1] * 125], 8)
