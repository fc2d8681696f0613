"""KV-cache serving on the Llama engine's weights: chunked prefill into a paged cache, batched one-token decode on
the split-K paged attention kernel, greedy sampling on the device.

`LlamaKVModel` is the model side of `serving.ServingScheduler.step`: the native scheduler (admission, block tables,
chunked prefill within a token budget, completion) hands it prompt chunks and the running sequences' newest tokens
together with their block tables, and gets next tokens back.  Nothing is recomputed: every token's K and V are
written once (`lt_kv_append`) and read by the attention of later tokens (`lt_paged_decode`, `lt_flash_fwd` for a
prompt chunk).  The reference's counterparts: ContinuousBatchingScheduler::step and its block tables
(src/llm/continuous_batching.cpp:20-197), paged attention (src/ops/attention.cpp:351-477) and flash-decoding
(src/ops/flash_decoding.cpp:13-115); its cache is never filled, here `PagedKVCache.append` is the write path.
"""
from __future__ import annotations

from collections import OrderedDict
from typing import List, Sequence

import torch

from ..serving import PagedKVCache
from .llama import LlamaEngine


class LlamaKVModel:
    def __init__(self, engine: LlamaEngine, num_blocks: int, block_size: int = 16, kv_dtype=torch.bfloat16, num_splits: int = 0,
                 graphs: bool = True, prefix_cache_bytes: int = 0):
        assert engine.w.tp == 1 and hasattr(engine.w, "flat_p"), "serving runs on whole (unsharded) weights"
        self.e = engine
        cfg = engine.cfg
        self.block_size = block_size
        self.num_splits = num_splits
        self.graphs = graphs                 # record the decode step per (batch size, table width) and replay it
        self._graphs = {}
        self.sampler = None                  # None: greedy on the device; else a callable logits [rows, vocab] -> tokens
        self.cache = PagedKVCache(cfg.n_layers, num_blocks, block_size, cfg.n_kv_heads, cfg.head_dim, device=engine.device,
                                  dtype=kv_dtype)
        self.kv_bytes_per_token = 2 * cfg.n_layers * cfg.n_kv_heads * cfg.head_dim * self.cache.k[0].element_size()
        # ---- prefix reuse: K / V of finished prompts' whole blocks are kept as snapshots (up to `prefix_cache_bytes`,
        # least recently used first out); a later prompt that starts with the same tokens gets those blocks by a copy
        # and only its remaining tokens are computed.  The reference has the prefix map (src/llm/prefix_cache.cpp) but
        # never consults it while serving.
        self.prefix_cache_bytes = int(prefix_cache_bytes)
        self.prefill_tokens_computed = 0
        self.prefill_tokens_reused = 0
        self._snap = OrderedDict()           # handle -> (k [layers, nb, Hkv, bs, hd], v, bytes)
        self._snap_bytes = 0
        self._next_handle = 1
        self._seq_tokens = {}                # first block of a sequence in prefill -> its prompt tokens so far
        if self.prefix_cache_bytes > 0:
            from ..serving import PrefixCache
            self._index = PrefixCache()

    # ------------------------------------------------------------------ shared layer body
    def _layers(self, x, positions, attend):
        e, cfg, w, K = self.e, self.e.cfg, self.e.w, self.e.K
        Hq, Hkv, hd = cfg.n_heads, cfg.n_kv_heads, cfg.head_dim
        n = x.shape[0]
        for i in range(cfg.n_layers):
            p = "layers.%d." % i
            h, _, _, _ = K.norm_fwd(x, w.p(p + "attn_norm"), eps=cfg.rms_eps)
            qkv = K.gemm(h, w.p(p + "wqkv"))
            K.rope_(qkv, e.cos, e.sin, 1, Hq, hd, col_offset=0, positions=positions)
            K.rope_(qkv, e.cos, e.sin, 1, Hkv, hd, col_offset=Hq * hd, positions=positions)
            q = qkv[:, :Hq * hd].view(n, Hq, hd)
            k = qkv[:, Hq * hd:(Hq + Hkv) * hd].view(n, Hkv, hd)
            v = qkv[:, (Hq + Hkv) * hd:].view(n, Hkv, hd)
            o = attend(i, q, k, v)
            x1 = K.gemm(o.reshape(n, Hq * hd), w.p(p + "wo"), residual=x)
            h2, _, _, _ = K.norm_fwd(x1, w.p(p + "mlp_norm"), eps=cfg.rms_eps)
            hm = K.swiglu_fwd(K.gemm(h2, w.p(p + "w_gu")))
            x = K.gemm(hm, w.p(p + "w_down"), residual=x1)
        return x

    def _next_tokens(self, x_rows):
        e, K = self.e, self.e.K
        hf, _, _, _ = K.norm_fwd(x_rows, e.w.p("final_norm"), eps=e.cfg.rms_eps)
        logits = K.gemm(hf, e.w.p("lm_head"))
        self.last_logits = logits            # [rows, vocab] of the newest step (kept for inspection and tests)
        if self.sampler is not None:
            return self.sampler(logits.float())
        return logits.float().argmax(-1)

    def _slots(self, block_ids: Sequence[int], start: int, n: int) -> torch.Tensor:
        bs = self.block_size
        return torch.tensor([block_ids[p // bs] * bs + p % bs for p in range(start, start + n)], dtype=torch.int32)

    # ------------------------------------------------------------------ prompt chunks
    @torch.no_grad()
    def prefill_chunk(self, tokens: Sequence[int], start: int, block_ids: Sequence[int], want_token: bool) -> int:
        """Run prompt positions [start, start + len(tokens)) of one sequence: their K / V go into the sequence's blocks,
        their queries attend to everything cached so far.  Returns the greedy next token when `want_token` (the chunk
        completes the prompt), else -1."""
        if self.prefix_cache_bytes > 0:
            return self._prefill_with_reuse(list(tokens), start, block_ids, want_token)
        return self._prefill_compute(tokens, start, block_ids, want_token)

    # ---- prefix reuse around the computation
    def _prefill_with_reuse(self, tokens: List[int], start: int, block_ids: Sequence[int], want_token: bool) -> int:
        bs = self.block_size
        key = block_ids[0]
        sofar = (self._seq_tokens.get(key, []) if start > 0 else []) + tokens
        end = start + len(tokens)
        matched, handles = self._index.longest_prefix(sofar, bs)
        snap = self._snap.get(handles[0]) if handles else None
        covered = start
        if snap is not None and matched > start:
            self._snap.move_to_end(handles[0])
            m = min(matched, snap[0].shape[1] * bs)
            if m >= end and want_token:                           # the last token's logits are needed: compute it
                m = (end - 1) // bs * bs
            if m > start:
                b0, b1 = start // bs, m // bs
                dst = torch.tensor(list(block_ids[b0:b1]), dtype=torch.int64, device=self.e.device)
                for i in range(self.e.cfg.n_layers):
                    self.cache.k[i][dst] = snap[0][i, b0:b1]
                    self.cache.v[i][dst] = snap[1][i, b0:b1]
                self.prefill_tokens_reused += m - start
                covered = m
        out = self._prefill_compute(sofar[covered:end], covered, block_ids, want_token) if covered < end else -1
        if want_token:
            self._seq_tokens.pop(key, None)
            self._remember(sofar, block_ids)
        else:
            self._seq_tokens[key] = sofar
        return out

    def _remember(self, prompt: List[int], block_ids: Sequence[int]) -> None:
        bs = self.block_size
        nb = len(prompt) // bs
        if nb == 0:
            return
        L = nb * bs
        got, handles = self._index.longest_prefix(prompt[:L], bs)
        if got == L and handles and handles[0] in self._snap:
            return                                                # this prefix is cached already
        blocks = torch.tensor(list(block_ids[:nb]), dtype=torch.int64, device=self.e.device)
        k = torch.stack([self.cache.k[i][blocks] for i in range(self.e.cfg.n_layers)])
        v = torch.stack([self.cache.v[i][blocks] for i in range(self.e.cfg.n_layers)])
        nbytes = 2 * k.numel() * k.element_size()
        if nbytes > self.prefix_cache_bytes:
            return
        while self._snap and self._snap_bytes + nbytes > self.prefix_cache_bytes:
            _, (_, _, old) = self._snap.popitem(last=False)
            self._snap_bytes -= old
        h = self._next_handle
        self._next_handle += 1
        self._snap[h] = (k, v, nbytes)
        self._snap_bytes += nbytes
        # findable by prompts that share the whole thing or a power-of-two number of its blocks: a later prompt reuses at
        # least half of the whole blocks it shares, for a logarithmic number of index entries per prompt
        lengths, j = {L}, 1
        while j * bs < L:
            lengths.add(j * bs)
            j *= 2
        from ..serving import _i32
        for n in sorted(lengths):                                 # the native index alone (it evicts by itself)
            self._index._lib.lt_prefix_insert(self._index._c, _i32(prompt[:n]), n, _i32([h]), 1)

    @torch.no_grad()
    def _prefill_compute(self, tokens: Sequence[int], start: int, block_ids: Sequence[int], want_token: bool) -> int:
        e, K = self.e, self.e.K
        dev = e.device
        n = len(tokens)
        self.prefill_tokens_computed += n
        host = torch.empty(3, n, dtype=torch.int64)
        host[0] = torch.tensor(tokens, dtype=torch.int64)
        host[1] = torch.arange(start, start + n)
        host[2] = self._slots(block_ids, start, n)
        d = host.to(dev, non_blocking=True)
        tok, pos, slots = d[0], d[1].to(torch.int32), d[2].to(torch.int32)
        bs = self.block_size
        nb = (start + n + bs - 1) // bs
        blocks = torch.tensor(list(block_ids[:nb]), dtype=torch.int64, device=dev) if start > 0 else None

        def attend(i, q, k, v):
            self.cache.append(i, k.contiguous(), v.contiguous(), slots)
            if start == 0:
                o, _ = K.flash_fwd(q.unsqueeze(0), k.unsqueeze(0), v.unsqueeze(0), causal=True)
                return o[0]
            # later chunk: keys and values of the whole context so far, read back from the sequence's blocks
            Hkv, hd = k.shape[1], k.shape[2]
            kc = self.cache.k[i][blocks].permute(0, 2, 1, 3).reshape(nb * bs, Hkv, hd)[:start + n]
            vc = self.cache.v[i][blocks].permute(0, 2, 1, 3).reshape(nb * bs, Hkv, hd)[:start + n]
            if self.cache.fp8:
                kc = (kc.float() * self.cache.k_scale).to(q.dtype)
                vc = (vc.float() * self.cache.v_scale).to(q.dtype)
            o, _ = K.flash_fwd(q.unsqueeze(0), kc.contiguous().unsqueeze(0), vc.contiguous().unsqueeze(0), causal=True)
            return o[0]

        x = self._layers(K.embedding_fwd(tok, e.w.p("embed")), pos, attend)
        if not want_token:
            return -1
        return int(self._next_tokens(x[-1:]).item())

    # ------------------------------------------------------------------ one token for every running sequence
    def _decode_body(self, d: torch.Tensor, S: int, width: int) -> torch.Tensor:
        """The device work of one decode step on the packed int64 input block `d` [4 + width, S]: rows 0-3 are token,
        position, cache slot and context length of every sequence, the rest its block table (transposed)."""
        from ..serving import paged_attention
        e, K = self.e, self.e.K
        bs = self.block_size
        tok = d[0]
        pos, slots, ctx = d[1].to(torch.int32), d[2].to(torch.int32), d[3].to(torch.int32)
        bt = d[4:].t().contiguous().to(torch.int32)
        splits = self.num_splits or self._splits(S, width * bs)

        def attend(i, q, k, v):
            self.cache.append(i, k.contiguous(), v.contiguous(), slots)
            return paged_attention(q.contiguous(), self.cache.k[i], self.cache.v[i], bt, ctx, bs, num_splits=splits,
                                   k_scale=self.cache.k_scale, v_scale=self.cache.v_scale)

        x = self._layers(K.embedding_fwd(tok, e.w.p("embed")), pos, attend)
        return self._next_tokens(x)

    @torch.no_grad()
    def decode_batch(self, last_tokens: Sequence[int], positions: Sequence[int], block_tables: List[Sequence[int]]) -> List[int]:
        """last_tokens[s] sits at position positions[s] of sequence s and is not in the cache yet: append its K / V,
        attend over positions[s] + 1 cached keys, return the greedy next token of every sequence.

        On a GPU the step's ~270 launches are recorded once per (batch size, block-table width) into a CUDA graph and
        replayed: the step then costs its kernels, not their launch overhead.  The inputs of a replay are copied
        into the graph's static input block first."""
        e = self.e
        dev = e.device
        S = len(last_tokens)
        bs = self.block_size
        width = max((p + bs) // bs for p in positions)
        if self.graphs and dev.type == "cuda":
            width = (width + 15) // 16 * 16                     # fewer distinct graphs: table widths in steps of 16 blocks
        host = torch.zeros(4 + width, S, dtype=torch.int64)
        host[0] = torch.tensor(list(last_tokens), dtype=torch.int64)
        host[1] = torch.tensor(list(positions), dtype=torch.int64)
        for s in range(S):
            p = positions[s]
            host[2, s] = block_tables[s][p // bs] * bs + p % bs
            row = block_tables[s][:width]
            host[4:4 + len(row), s] = torch.tensor(list(row), dtype=torch.int64)
        host[3] = host[1] + 1
        if not (self.graphs and dev.type == "cuda"):
            return self._decode_body(host.to(dev, non_blocking=True), S, width).tolist()
        key = (S, width)
        entry = self._graphs.get(key)
        if entry is None:
            static_in = host.to(dev)
            side = torch.cuda.Stream(device=dev)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):                        # eager run on the capture stream: workspaces, caches
                self._decode_body(static_in, S, width)
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                static_out = self._decode_body(static_in, S, width)
            entry = self._graphs[key] = (g, static_in, static_out)
            # the two recording passes appended this step's K / V already; the replay below rewrites the same slots
        g, static_in, static_out = entry
        static_in.copy_(host, non_blocking=True)
        g.replay()
        return static_out.tolist()

    def _splits(self, S: int, max_ctx: int) -> int:
        """Splits of the key range per (sequence, KV head): about four CTAs per SM, at least 256 keys per split."""
        ctas = S * self.e.cfg.n_kv_heads
        return max(1, min(32, max_ctx // 256, (148 * 4 + ctas - 1) // ctas))


class Sampler:
    """Temperature / top-k / nucleus sampling of next tokens from logits [rows, vocab] with its own random generator, so
    that a run is reproducible from its seed.  `temperature == 0` (or `top_k == 1`) is greedy."""

    def __init__(self, temperature: float = 1.0, top_k: int = 0, top_p: float = 1.0, seed: int = 0, device="cpu"):
        self.temperature, self.top_k, self.top_p = float(temperature), int(top_k), float(top_p)
        self.gen = torch.Generator(device=device).manual_seed(int(seed))

    def __call__(self, logits: torch.Tensor) -> torch.Tensor:
        if self.temperature <= 0.0 or self.top_k == 1:
            return logits.argmax(-1)
        z = logits / self.temperature
        if self.top_k > 0 and self.top_k < z.shape[-1]:
            kth = z.topk(self.top_k, -1).values[..., -1:]
            z = z.masked_fill(z < kth, float("-inf"))
        if self.top_p < 1.0:
            order = z.sort(-1, descending=True)
            p = torch.softmax(order.values, -1)
            before = p.cumsum(-1) - p                     # probability mass ahead of each token, in sorted order
            drop = before >= self.top_p                   # the first token always stays
            z = z.masked_fill(torch.zeros_like(drop).scatter(-1, order.indices, drop), float("-inf"))
        return torch.multinomial(torch.softmax(z, -1), 1, generator=self.gen).squeeze(-1)


@torch.no_grad()
def generate(engine: LlamaEngine, prompts: Sequence[Sequence[int]], max_new_tokens: int, *, temperature: float = 0.0,
             top_k: int = 0, top_p: float = 1.0, seed: int = 0, eos_id: int = -1, block_size: int = 16,
             max_num_seqs: int = 64, max_num_batched_tokens: int = 4096, kv_dtype=None,
             prefix_cache_bytes: int = 0) -> List[List[int]]:
    """Continue every prompt by up to `max_new_tokens` tokens (stopping at `eos_id`) with continuous batching on a paged KV
    cache sized for the request, and return the new tokens per prompt.  Greedy by default (the decode step is replayed
    from CUDA graphs on a GPU); with `temperature > 0` the next tokens are drawn by `Sampler` (eager decode steps)."""
    from ..serving import Request, ServingScheduler
    cfg = engine.cfg
    need = sum((len(p) + max_new_tokens + block_size - 1) // block_size for p in prompts)
    greedy = temperature <= 0.0 or top_k == 1
    if kv_dtype is None:
        kv_dtype = torch.bfloat16 if engine.device.type == "cuda" else torch.float32
    model = LlamaKVModel(engine, num_blocks=need + 1, block_size=block_size, kv_dtype=kv_dtype, graphs=greedy,
                         prefix_cache_bytes=prefix_cache_bytes)   # prompts of one call that share a prefix reuse its blocks
    if not greedy:
        model.sampler = Sampler(temperature, top_k, top_p, seed, device=engine.device)
    sched = ServingScheduler(num_blocks=need + 1, block_size=block_size, max_num_seqs=max_num_seqs,
                             max_num_batched_tokens=max_num_batched_tokens, eos_id=eos_id)
    reqs = [Request(i, list(p), max_new_tokens=max_new_tokens) for i, p in enumerate(prompts)]
    for r in reqs:
        if len(r.prompt_tokens) + max_new_tokens > cfg.max_seq:
            raise ValueError("prompt %d: %d tokens + %d new exceed the model's %d positions" %
                             (r.id, len(r.prompt_tokens), max_new_tokens, cfg.max_seq))
        sched.add_request(r)
    finished, guard = 0, 0
    while finished < len(reqs):
        finished += len(sched.step(model))
        guard += 1
        if guard > 4 * (max_new_tokens + len(reqs)) + 64 + sum(len(p) for p in prompts):
            raise RuntimeError("the schedule did not finish")
    return [list(r.generated_tokens) for r in reqs]
