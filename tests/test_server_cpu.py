"""The HTTP front end on the CPU: concurrent clients share the running batch, every answer equals greedy decoding by full
recomputation, bad requests are refused with 400, and finished requests leave no state behind."""
import json
import threading
import urllib.error
import urllib.request

import torch


def _post(port, obj):
    req = urllib.request.Request("http://127.0.0.1:%d/generate" % port, data=json.dumps(obj).encode(),
                                 headers={"Content-Type": "application/json"})
    with urllib.request.urlopen(req, timeout=120) as r:
        return json.loads(r.read())


def test_concurrent_http_clients_get_the_greedy_continuations():
    from litetorch_b200 import server
    from litetorch_b200.models.llama import LlamaConfig, LlamaEngine, LocalWeights
    from litetorch_b200.models.llama_serving import LlamaKVModel
    cfg = LlamaConfig.tiny()
    engine = LlamaEngine(cfg, "cpu", weights=LocalWeights(cfg, "cpu", seed=4, param_dtype=torch.float32))
    model = LlamaKVModel(engine, num_blocks=96, block_size=8, kv_dtype=torch.float32)
    encode, decode, _ = server.tokenizer()
    loop = server.EngineLoop(model, 96, 8, max_num_seqs=4, max_num_batched_tokens=32, eos_id=-1, max_context=cfg.max_seq)
    httpd = server.serve(loop, encode, decode, port=0)
    port = httpd.server_address[1]
    try:
        g = torch.Generator().manual_seed(0)
        prompts = [torch.randint(3, cfg.vocab_size, (n,), generator=g).tolist() for n in (5, 23, 40, 9, 17, 31)]
        answers = [None] * len(prompts)

        def client(i):
            answers[i] = _post(port, {"prompt_ids": prompts[i], "max_new_tokens": 3 + i % 3})
        threads = [threading.Thread(target=client, args=(i,)) for i in range(len(prompts))]
        for t in threads:
            t.start()
        for t in threads:
            t.join(timeout=300)
        for i, (p, a) in enumerate(zip(prompts, answers)):
            assert a is not None and a["new_tokens"] == 3 + i % 3 and a["prompt_tokens"] == len(p)
            ctx = list(p)
            for tok in a["ids"]:
                assert int(engine.forward_logits(torch.tensor([ctx]))[0, -1].argmax()) == tok
                ctx.append(tok)
        assert _post(port, {"prompt": "5,6,7", "max_new_tokens": 2})["text"].count(",") == 1      # the text form of ids
        # streaming: pieces arrive as JSON lines and concatenate to the non-streamed answer
        req = urllib.request.Request("http://127.0.0.1:%d/generate" % port, headers={"Content-Type": "application/json"},
                                     data=json.dumps({"prompt_ids": prompts[1], "max_new_tokens": 5, "stream": True}).encode())
        with urllib.request.urlopen(req, timeout=120) as r:
            lines = [json.loads(l) for l in r.read().decode().splitlines()]
        assert lines[-1]["done"] and lines[-1]["new_tokens"] == 5 and len(lines) >= 3
        streamed = [t for l in lines[:-1] for t in l["ids"]]
        assert streamed == _post(port, {"prompt_ids": prompts[1], "max_new_tokens": 5})["ids"]
        assert [t for piece in loop.stream(prompts[0], 3) for t in piece] == answers[0]["ids"]
        health = json.loads(urllib.request.urlopen("http://127.0.0.1:%d/health" % port, timeout=30).read())
        assert health == {"running": 0, "pending": 0, "free_blocks": 96, "served": 10}
        metrics = urllib.request.urlopen("http://127.0.0.1:%d/metrics" % port, timeout=30).read().decode()
        assert "litetorch_served 10" in metrics and "# TYPE litetorch_free_blocks gauge" in metrics
        assert "litetorch_prefill_tokens_computed" in metrics
        assert not loop.sched._reqs and not loop.sched._order                      # nothing is kept for finished requests
        for bad in ({"max_new_tokens": 4}, {"prompt_ids": [], "max_new_tokens": 4}, {"prompt_ids": [1] * 250, "max_new_tokens": 50}):
            try:
                _post(port, bad)
                raise AssertionError("accepted %r" % (bad,))
            except urllib.error.HTTPError as e:
                assert e.code == 400
    finally:
        httpd.shutdown()
        loop.close()
