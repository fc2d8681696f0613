"""The engine on the device with weights converted from a Hugging Face Llama: logits against `transformers`' forward pass
in fp32 on the same bf16-rounded weights, and greedy generation through the paged KV cache against the engine's own
full-recompute logits."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_engine_logits_follow_the_hugging_face_model_on_the_device():
    transformers = pytest.importorskip("transformers")
    from transformers import LlamaConfig as HC, LlamaForCausalLM
    from litetorch_b200.models import llama_io
    from litetorch_b200.models.llama import LlamaEngine
    from litetorch_b200.models.llama_serving import generate
    from litetorch_b200.ops import kernels as K
    torch.manual_seed(0)
    hc = HC(vocab_size=512, hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
            num_key_value_heads=2, head_dim=64, max_position_embeddings=256, rms_norm_eps=1e-5, rope_theta=10000.0,
            tie_word_embeddings=False, attention_bias=False, mlp_bias=False)
    model = LlamaForCausalLM(hc).eval().float()
    with torch.no_grad():
        for p in model.parameters():
            p.copy_(p.to(torch.bfloat16).float())          # both sides compute with the same rounded weights
    cfg = llama_io.config_from_hf(hc)
    engine = LlamaEngine(cfg, "cuda", seed=1)
    llama_io.load_into(engine, model.state_dict())
    tok = torch.randint(0, cfg.vocab_size, (2, 200), generator=torch.Generator().manual_seed(3))
    with torch.no_grad():
        ref = model(tok).logits
    got = engine.forward_logits(tok.cuda()).float().cpu()
    torch.cuda.synchronize()
    K.check_status()
    assert float((got - ref).abs().max()) < 3e-2 * max(1.0, float(ref.abs().max()))
    # generation through the paged cache picks, at every step, a token whose full-recompute logit is (nearly) the largest
    prompts = [tok[0, :37].tolist(), tok[1, :90].tolist()]
    outs = generate(engine, prompts, 6)
    for p, o in zip(prompts, outs):
        ctx = list(p)
        for t in o:
            row = engine.forward_logits(torch.tensor([ctx], device="cuda"))[0, -1].float()
            assert float(row.max() - row[t]) < 5e-2
            ctx.append(t)
