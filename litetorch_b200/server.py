"""A small HTTP front end for the serving path: one engine thread runs `ServingScheduler.step(model)` in a loop
(continuous batching: requests join and leave the running batch between steps), handler threads add requests and wait
for theirs to finish.  Standard library only.

    python -m litetorch_b200.server --model /models/llama --port 8000 [--sentencepiece tok.model | --bytes]

    POST /generate   {"prompt": "text" | "prompt_ids": [1, 2, 3], "max_new_tokens": 32, "stream": false}
                  -> {"ids": [...], "text": "...", "prompt_tokens": n, "new_tokens": m, "seconds": s}
                     with "stream": true, one JSON line per piece as the tokens arrive, then {"done": true, ...}
    GET  /health     {"running": r, "pending": p, "free_blocks": f, "served": n}
    GET  /metrics    the same counters and the prefill token counts in the Prometheus text format

Decoding is greedy (the decode step is replayed from CUDA graphs on a GPU).  The reference has the scheduler and no
server around it (src/llm/continuous_batching.cpp); `EngineLoop` is that missing piece and is usable without HTTP:
`loop.submit(prompt_ids, max_new_tokens)` returns the finished `Request`.
"""
from __future__ import annotations

import argparse
import itertools
import json
import threading
import time
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from typing import List, Optional, Sequence

from .serving import Request, ServingScheduler


class EngineLoop:
    """Owns the scheduler and the model; `submit` may be called from any thread."""

    def __init__(self, model, num_blocks: int, block_size: int = 16, max_num_seqs: int = 64,
                 max_num_batched_tokens: int = 4096, eos_id: int = -1, max_context: Optional[int] = None):
        self.model = model
        self.block_size, self.num_blocks, self.max_context = block_size, num_blocks, max_context
        self.sched = ServingScheduler(num_blocks, block_size, max_num_seqs, max_num_batched_tokens, eos_id)
        self._ids = itertools.count(1)
        self._lock = threading.Lock()              # the Python side of the scheduler (its request table) is not re-entrant
        self._wake = threading.Condition(self._lock)
        self._done = {}                            # request id -> Event
        self._live = {}                            # request id -> (Request, tokens already handed out, queue or None)
        self._stop = False
        self.served = 0
        self.error: Optional[BaseException] = None
        self._thread = threading.Thread(target=self._run, name="lt-engine-loop", daemon=True)
        self._thread.start()

    def _run(self):
        try:
            dev = getattr(getattr(self.model, "e", None), "device", None)
            if dev is not None and dev.type == "cuda" and dev.index is not None:
                import torch
                torch.cuda.set_device(dev)                      # the current device is per thread
            while True:
                with self._wake:
                    while not self._stop and not self._done:
                        self._wake.wait()
                    if self._stop:
                        return
                    finished = self.sched.step(self.model)     # one step under the lock: submissions wait at most a step
                    for rid, (req, seen, q) in list(self._live.items()):
                        if q is not None and len(req.generated_tokens) > seen:        # streaming: hand out the new tokens
                            q.put(list(req.generated_tokens[seen:]))
                            self._live[rid] = (req, len(req.generated_tokens), q)
                    for r in finished:
                        ev = self._done.pop(r.id, None)
                        _, _, q = self._live.pop(r.id, (None, 0, None))
                        if q is not None:
                            q.put(None)                        # end of stream
                        self.served += 1
                        if ev is not None:
                            ev.set()
        except BaseException as e:                              # a failed step must not leave the waiters hanging
            self.error = e
            with self._wake:
                for ev in self._done.values():
                    ev.set()
                for _, _, q in self._live.values():
                    if q is not None:
                        q.put(None)
                self._done.clear()
                self._live.clear()

    def _check(self, prompt_ids, max_new_tokens):
        need = (len(prompt_ids) + max_new_tokens + self.block_size - 1) // self.block_size
        if not prompt_ids or max_new_tokens < 1:
            raise ValueError("a request needs a prompt and at least one new token")
        if need > self.num_blocks or (self.max_context and len(prompt_ids) + max_new_tokens > self.max_context):
            raise ValueError("the request does not fit: %d prompt + %d new tokens" % (len(prompt_ids), max_new_tokens))
        if self.error is not None:
            raise RuntimeError("the engine loop stopped: %r" % (self.error,))

    def _enqueue(self, prompt_ids, max_new_tokens, q):
        ev = threading.Event()
        with self._wake:
            req = Request(next(self._ids), list(prompt_ids), max_new_tokens=max_new_tokens)
            self.sched.add_request(req)
            self._done[req.id] = ev
            self._live[req.id] = (req, 0, q)
            self._wake.notify_all()
        return req, ev

    def stream(self, prompt_ids: Sequence[int], max_new_tokens: int, timeout_s: float = 600.0):
        """Yields lists of new token ids as the engine produces them (one list per scheduling step that advanced the
        request), then returns."""
        import queue
        self._check(prompt_ids, max_new_tokens)
        q = queue.Queue()
        self._enqueue(prompt_ids, max_new_tokens, q)
        while True:
            try:
                item = q.get(timeout=timeout_s)
            except queue.Empty:
                raise TimeoutError("the stream stalled for %.0f s" % timeout_s)
            if item is None:
                break
            yield item
        if self.error is not None:
            raise RuntimeError("the engine loop stopped: %r" % (self.error,))

    def submit(self, prompt_ids: Sequence[int], max_new_tokens: int, timeout_s: float = 600.0) -> Request:
        self._check(prompt_ids, max_new_tokens)
        req, ev = self._enqueue(prompt_ids, max_new_tokens, None)
        if not ev.wait(timeout_s):
            raise TimeoutError("request %d did not finish in %.0f s" % (req.id, timeout_s))
        if self.error is not None:
            raise RuntimeError("the engine loop stopped: %r" % (self.error,))
        return req

    def stats(self) -> dict:
        with self._lock:
            return {"running": len(self.sched.running_queue), "pending": len(self.sched.pending_queue),
                    "free_blocks": int(self.sched.free_blocks), "served": self.served}

    def close(self):
        with self._wake:
            self._stop = True
            self._wake.notify_all()
        self._thread.join(timeout=30)


def make_handler(loop: EngineLoop, encode, decode, default_new: int = 32):
    class Handler(BaseHTTPRequestHandler):
        def _send(self, code: int, obj: dict):
            body = json.dumps(obj).encode()
            self.send_response(code)
            self.send_header("Content-Type", "application/json")
            self.send_header("Content-Length", str(len(body)))
            self.end_headers()
            self.wfile.write(body)

        def log_message(self, *a):                              # quiet: one line per request is the caller's business
            pass

        def _stream(self, ids, max_new, t0):
            """One JSON object per line as tokens arrive ({"ids", "text"}), a closing line with the totals."""
            pieces = loop.stream(ids, max_new)
            first = next(pieces, None)                          # validation errors surface before the headers are sent
            self.send_response(200)
            self.send_header("Content-Type", "application/x-ndjson")
            self.send_header("Connection", "close")
            self.end_headers()
            total = 0
            while first is not None:
                total += len(first)
                self.wfile.write((json.dumps({"ids": first, "text": decode(first)}) + "\n").encode())
                self.wfile.flush()
                first = next(pieces, None)
            self.wfile.write((json.dumps({"done": True, "prompt_tokens": len(ids), "new_tokens": total,
                                          "seconds": round(time.time() - t0, 4)}) + "\n").encode())

        def do_GET(self):
            if self.path == "/health":
                return self._send(200, loop.stats())
            if self.path == "/metrics":                         # Prometheus text exposition format
                st = loop.stats()
                model = loop.model
                st["prefill_tokens_computed"] = getattr(model, "prefill_tokens_computed", 0)
                st["prefill_tokens_reused"] = getattr(model, "prefill_tokens_reused", 0)
                kinds = {"served": "counter", "prefill_tokens_computed": "counter", "prefill_tokens_reused": "counter"}
                body = "".join("# TYPE litetorch_%s %s\nlitetorch_%s %d\n" % (k, kinds.get(k, "gauge"), k, int(v))
                               for k, v in sorted(st.items())).encode()
                self.send_response(200)
                self.send_header("Content-Type", "text/plain; version=0.0.4")
                self.send_header("Content-Length", str(len(body)))
                self.end_headers()
                self.wfile.write(body)
                return
            self._send(404, {"error": "unknown path"})

        def do_POST(self):
            if self.path != "/generate":
                return self._send(404, {"error": "unknown path"})
            try:
                req = json.loads(self.rfile.read(int(self.headers.get("Content-Length", "0"))) or b"{}")
                ids = [int(t) for t in req["prompt_ids"]] if "prompt_ids" in req else encode(str(req["prompt"]))
                t0 = time.time()
                if req.get("stream"):
                    return self._stream(ids, int(req.get("max_new_tokens", default_new)), t0)
                done = loop.submit(ids, int(req.get("max_new_tokens", default_new)))
                out = list(done.generated_tokens)
                self._send(200, {"ids": out, "text": decode(out), "prompt_tokens": len(ids), "new_tokens": len(out),
                                 "seconds": round(time.time() - t0, 4)})
            except (KeyError, ValueError, TypeError) as e:
                self._send(400, {"error": str(e)})
            except Exception as e:                              # engine failure or timeout
                self._send(500, {"error": repr(e)})
    return Handler


def serve(loop: EngineLoop, encode, decode, host: str = "127.0.0.1", port: int = 8000) -> ThreadingHTTPServer:
    """Start the HTTP server on a background thread and return it (`.shutdown()` stops it; port 0 picks a free one)."""
    httpd = ThreadingHTTPServer((host, port), make_handler(loop, encode, decode))
    threading.Thread(target=httpd.serve_forever, name="lt-http", daemon=True).start()
    return httpd


def tokenizer(sentencepiece: str = "", byte_level: bool = False):
    """(encode, decode, eos_id) for a SentencePiece model, byte-level ids, or comma-separated ids."""
    if sentencepiece:
        import sentencepiece as spm
        sp = spm.SentencePieceProcessor(model_file=sentencepiece)
        return (lambda s: [sp.bos_id()] * (sp.bos_id() >= 0) + sp.encode(s)), sp.decode, sp.eos_id()
    if byte_level:
        return (lambda s: list(s.encode("utf-8"))), (lambda ids: bytes(i for i in ids if i < 256).decode("utf-8", "replace")), 256
    return (lambda s: [int(t) for t in s.split(",")]), (lambda ids: ",".join(str(i) for i in ids)), -1


def main(argv=None):
    import torch
    from .models import llama_io
    from .models.llama_serving import LlamaKVModel
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", required=True, help="Hugging Face directory (config.json + *.safetensors)")
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--sentencepiece", default="")
    ap.add_argument("--bytes", action="store_true")
    ap.add_argument("--device", default="cuda")
    ap.add_argument("--kv-blocks", type=int, default=4096)
    ap.add_argument("--block-size", type=int, default=16)
    ap.add_argument("--max-num-seqs", type=int, default=64)
    ap.add_argument("--max-batched-tokens", type=int, default=4096)
    ap.add_argument("--prefix-cache-mb", type=int, default=0, help="keep K / V of finished prompts for reuse by prompts that share a prefix")
    args = ap.parse_args(argv)
    kw = {}
    if args.device == "cpu":
        import os
        from .models.llama import LocalWeights
        with open(os.path.join(args.model, "config.json")) as f:
            cfg = llama_io.config_from_hf(json.load(f))
        kw["weights"] = LocalWeights(cfg, "cpu", seed=0, param_dtype=torch.float32)
    engine = llama_io.load_pretrained(args.model, device=args.device, **kw)
    model = LlamaKVModel(engine, num_blocks=args.kv_blocks, block_size=args.block_size,
                         kv_dtype=torch.float32 if args.device == "cpu" else torch.bfloat16,
                         prefix_cache_bytes=args.prefix_cache_mb << 20)
    encode, decode, eos = tokenizer(args.sentencepiece, args.bytes)
    loop = EngineLoop(model, args.kv_blocks, args.block_size, args.max_num_seqs, args.max_batched_tokens, eos_id=eos,
                      max_context=engine.cfg.max_seq)
    httpd = serve(loop, encode, decode, args.host, args.port)
    print("serving %s on http://%s:%d" % (args.model, args.host, httpd.server_address[1]), flush=True)
    try:
        while True:
            time.sleep(3600)
    except KeyboardInterrupt:
        pass
    finally:
        httpd.shutdown()
        loop.close()


if __name__ == "__main__":
    main()
