"""Serving: paged KV cache, continuous batching, prefix cache, speculative / Medusa decoding, guided decoding.

The scheduler, block manager, token-prefix cache and the guided-decoding mask are native (C++,
csrc/runtime/scheduler.cpp); the decode attention and the KV-append are CUDA kernels
(csrc/kernels/paged_decode.cu).  Class and method names follow the reference binding
(src/bindings/python_bindings.cpp:530-584): `Request`, `ServingScheduler.{add_request, step,
get_block_table_tensor, get_context_lens_tensor}`, `PrefixCache.get().{put, get_cache, clear}`,
`SpeculativeEngine.generate`, `MedusaHead`, `MedusaEngine.generate`, `GuidedDecoder.apply_mask`.
Unlike the reference, which never fills `k_cache` / `v_cache`, `PagedKVCache.append` is the write path.
"""
from __future__ import annotations

import ctypes
from ctypes import c_int, c_int32, c_int64, c_void_p, c_char_p, c_uint8, POINTER
from typing import Dict, List, Optional, Sequence

import torch

from ._native import host_lib
from .core import Tensor, _unwrap

EOS_ID = 2


def _h():
    lib = host_lib()
    if not getattr(lib, "_lt_sched_bound", False):
        lib.lt_sched_create.restype = c_void_p
        lib.lt_sched_create.argtypes = [c_int] * 5
        lib.lt_sched_destroy.argtypes = [c_void_p]
        lib.lt_sched_add_request.argtypes = [c_void_p, c_int64, POINTER(c_int32), c_int, c_int]
        lib.lt_sched_plan.argtypes = [c_void_p, POINTER(c_int64), POINTER(c_int32), POINTER(c_int32), c_int]
        lib.lt_sched_commit.argtypes = [c_void_p, c_int64, c_int32]
        lib.lt_sched_tokens.argtypes = [c_void_p, c_int64, POINTER(c_int32), c_int, POINTER(c_int)]
        lib.lt_sched_block_table.argtypes = [c_void_p, c_int64, POINTER(c_int32), c_int]
        lib.lt_sched_context_len.argtypes = [c_void_p, c_int64]
        lib.lt_sched_pop_finished.argtypes = [c_void_p, POINTER(c_int64), c_int]
        lib.lt_sched_release.argtypes = [c_void_p, c_int64]
        for f in ("lt_sched_num_free_blocks", "lt_sched_num_running", "lt_sched_num_pending"):
            getattr(lib, f).argtypes = [c_void_p]
        lib.lt_prefix_create.restype = c_void_p
        lib.lt_prefix_create.argtypes = [c_int]
        lib.lt_prefix_destroy.argtypes = [c_void_p]
        lib.lt_prefix_insert.argtypes = [c_void_p, POINTER(c_int32), c_int, POINTER(c_int32), c_int]
        lib.lt_prefix_lookup.argtypes = [c_void_p, POINTER(c_int32), c_int, c_int, POINTER(c_int32), c_int, POINTER(c_int)]
        lib.lt_prefix_size.argtypes = [c_void_p]
        lib.lt_guided_mask.argtypes = [c_char_p, c_char_p, c_char_p, POINTER(c_int64), c_int, POINTER(c_uint8)]
        lib._lt_sched_bound = True
    return lib


def _i32(vals):
    return (c_int32 * len(vals))(*[int(v) for v in vals])


# ------------------------------------------------------------------------------------------------ paged KV cache
class PagedKVCache:
    """K/V blocks [num_blocks, Hkv, block_size, D] per layer, bf16 or e4m3 with per-tensor scales."""

    def __init__(self, num_layers: int, num_blocks: int, block_size: int, n_kv_heads: int, head_dim: int, device="cuda",
                 dtype=torch.bfloat16, k_scale: float = 1.0, v_scale: float = 1.0):
        self.block_size, self.n_kv_heads, self.head_dim = block_size, n_kv_heads, head_dim
        self.fp8 = dtype == torch.float8_e4m3fn
        self.k_scale, self.v_scale = k_scale, v_scale
        shape = (num_blocks, n_kv_heads, block_size, head_dim)
        self.k = [torch.zeros(shape, dtype=dtype, device=device) for _ in range(num_layers)]
        self.v = [torch.zeros(shape, dtype=dtype, device=device) for _ in range(num_layers)]

    def append(self, layer: int, k_new: torch.Tensor, v_new: torch.Tensor, slots: torch.Tensor):
        """k_new / v_new: [N, Hkv, D]; slots: [N] int32 = block * block_size + offset."""
        kc, vc = self.k[layer], self.v[layer]
        if kc.is_cuda:
            from .ops import kernels as K
            K.kv_append(k_new.contiguous(), v_new.contiguous(), kc, vc, slots.to(torch.int32), self.block_size, self.fp8,
                        self.k_scale, self.v_scale)
            return
        blk, off = slots.long() // self.block_size, slots.long() % self.block_size
        kq = k_new.float() / self.k_scale if self.fp8 else k_new
        vq = v_new.float() / self.v_scale if self.fp8 else v_new
        kc[blk, :, off] = kq.to(kc.dtype)
        vc[blk, :, off] = vq.to(vc.dtype)


def paged_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_tables: torch.Tensor,
                    context_lens: torch.Tensor, block_size: int, scale: Optional[float] = None, num_splits: int = 0,
                    k_scale: float = 1.0, v_scale: float = 1.0) -> torch.Tensor:
    """Decode attention of q [S, H, D] over paged caches [blocks, Hkv, block_size, D]; block tables and context
    lengths may be float tensors (reference convention).  CUDA bf16 queries use the split-K kernel."""
    S, H, D = q.shape
    Hkv = k_cache.shape[1]
    scale = (D ** -0.5) if scale is None else scale
    bt = block_tables.to(torch.int32).contiguous()
    cl = context_lens.to(torch.int32).contiguous()
    if q.is_cuda and q.dtype == torch.bfloat16 and D in (64, 128) and k_cache.dtype in (torch.bfloat16, torch.float8_e4m3fn):
        from .ops import kernels as K
        if num_splits <= 0:
            # about four CTAs (one per sequence, KV head and split) per SM, at least 256 keys per split
            max_ctx = int(cl.max().item()) if S else 0
            num_splits = max(1, min(32, max_ctx // 256, (148 * 4 + S * Hkv - 1) // max(S * Hkv, 1)))
        return K.paged_decode(q.contiguous(), k_cache, v_cache, bt, cl, block_size, num_splits, scale, k_scale, v_scale)
    out = torch.zeros(S, H, D, dtype=torch.float32, device=q.device)
    G = H // Hkv
    for s in range(S):
        n = int(cl[s])
        if n == 0:
            continue
        nb = (n + block_size - 1) // block_size
        blocks = bt[s, :nb].long()
        kk = k_cache[blocks].float().permute(1, 0, 2, 3).reshape(Hkv, nb * block_size, D)[:, :n] * k_scale
        vv = v_cache[blocks].float().permute(1, 0, 2, 3).reshape(Hkv, nb * block_size, D)[:, :n] * v_scale
        kk, vv = kk.repeat_interleave(G, 0), vv.repeat_interleave(G, 0)
        sc = torch.einsum("hd,htd->ht", q[s].float(), kk) * scale
        out[s] = torch.einsum("ht,htd->hd", torch.softmax(sc, -1), vv)
    return out.to(q.dtype)


# ------------------------------------------------------------------------------------------------ scheduler
class Request:
    def __init__(self, id: int, prompt: Sequence[int], max_new_tokens: int = 32):
        self.id = int(id)
        self.prompt_tokens = [int(t) for t in prompt]
        self.generated_tokens: List[int] = []
        self.max_new_tokens = int(max_new_tokens)
        self.prefill_processed = 0
        self.is_finished = False
        self.block_ids: List[int] = []


class _BlockCount(int):
    def __len__(self) -> int:
        return int(self)


class ServingScheduler:
    """Continuous batching over a paged KV pool.  `step(model)` admits, prefills in chunks within the token budget,
    decodes one token for every running sequence in ONE batched forward, samples greedily and returns the requests
    that finished in this step.  `model(tokens [B, T] as floats) -> logits [B, T, V]`."""

    def __init__(self, num_blocks: int, block_size: int, max_num_seqs: int, max_num_batched_tokens: int, eos_id: int = EOS_ID):
        self.num_blocks, self.block_size = num_blocks, block_size
        self.max_num_seqs, self.max_num_batched_tokens = max_num_seqs, max_num_batched_tokens
        self._lib = _h()
        self._s = self._lib.lt_sched_create(num_blocks, block_size, max_num_seqs, max_num_batched_tokens, eos_id)
        self._reqs: Dict[int, Request] = {}
        self._order: List[int] = []

    def __del__(self):
        try:
            self._lib.lt_sched_destroy(self._s)
        except Exception:
            pass

    def add_request(self, req: Request):
        if self._lib.lt_sched_add_request(self._s, req.id, _i32(req.prompt_tokens), len(req.prompt_tokens), req.max_new_tokens) != 0:
            raise ValueError("duplicate request id %d" % req.id)
        self._reqs[req.id] = req
        self._order.append(req.id)

    @property
    def pending_queue(self) -> List[Request]:
        n = self._lib.lt_sched_num_pending(self._s)
        waiting = [self._reqs[i] for i in self._order if not self._reqs[i].block_ids and not self._reqs[i].is_finished]
        return waiting[-n:] if n else []

    @property
    def running_queue(self) -> List[Request]:
        return [self._reqs[i] for i in self._order if self._reqs[i].block_ids and not self._reqs[i].is_finished]

    @property
    def free_blocks(self) -> "_BlockCount":
        """How many KV blocks are free.  The reference exposes the list of free block ids here and its callers take its length
        (tests/advanced_serving_test.cpp:84); the native scheduler keeps the ids to itself, so this is a count that also
        answers `len()`."""
        return _BlockCount(self._lib.lt_sched_num_free_blocks(self._s))

    def _sync(self, rid: int):
        r = self._reqs[rid]
        buf = (c_int32 * (len(r.prompt_tokens) + r.max_new_tokens + 8))()
        plen = c_int(0)
        n = self._lib.lt_sched_tokens(self._s, rid, buf, len(buf), ctypes.byref(plen))
        r.generated_tokens = [int(buf[i]) for i in range(plen.value, n)]
        bt = (c_int32 * 4096)()
        nb = self._lib.lt_sched_block_table(self._s, rid, bt, 4096)
        r.block_ids = [int(bt[i]) for i in range(min(nb, 4096))]
        r.prefill_processed = min(self._lib.lt_sched_context_len(self._s, rid), len(r.prompt_tokens))

    def _tokens(self, rid: int) -> List[int]:
        r = self._reqs[rid]
        return r.prompt_tokens + r.generated_tokens

    def step(self, model=None) -> List[Request]:
        """One scheduling step.  A model with `prefill_chunk` / `decode_batch` (e.g. `models.llama_serving.LlamaKVModel`)
        owns a paged KV cache and is driven with the scheduler's block tables: every token is computed once.  Any other
        callable `model(tokens) -> logits` is served by recomputing each context (the reference's behaviour).

        Without a model (the form the reference's serving guide shows) nothing is computed: pending requests are admitted
        while blocks are free and the requests that would run in this step are returned, so that the caller can read
        `get_block_table_tensor()` / `get_context_lens_tensor()` and drive its own kernels."""
        if model is None:
            cap = max(self.max_num_seqs, 1)
            ids, starts, lens = (c_int64 * cap)(), (c_int32 * cap)(), (c_int32 * cap)()
            n = self._lib.lt_sched_plan(self._s, ids, starts, lens, cap)      # planning alone changes no position
            for i in range(n):
                self._sync(int(ids[i]))
            return [self._reqs[int(ids[i])] for i in range(n)]
        if hasattr(model, "prefill_chunk") and hasattr(model, "decode_batch"):
            return self._step_kv(model)
        cap = max(self.max_num_seqs, 1)
        ids = (c_int64 * cap)()
        starts = (c_int32 * cap)()
        lens = (c_int32 * cap)()
        n = self._lib.lt_sched_plan(self._s, ids, starts, lens, cap)
        if n == 0:
            return []
        decode_ids = []
        for i in range(n):
            rid, st, ln = int(ids[i]), int(starts[i]), int(lens[i])
            self._sync(rid)
            if ln > 0:   # prefill chunk: one forward over the prompt seen so far, sample only when the prompt completes
                toks = self._reqs[rid].prompt_tokens[:st + ln]
                x = Tensor(torch.tensor([toks], dtype=torch.float32))
                logits = _unwrap(model(x))
                done = st + ln >= len(self._reqs[rid].prompt_tokens)
                nxt = int(logits[0, -1].float().argmax().item()) if done else -1
                self._lib.lt_sched_commit(self._s, rid, nxt)
            else:
                decode_ids.append(rid)
        if decode_ids:
            # Without a KV-cache-aware model the batched decode re-runs each context; sequences are right-aligned
            # by padding on the left so that position -1 is the newest token of every row.
            seqs = [self._tokens(r) for r in decode_ids]
            L = max(len(s) for s in seqs)
            batch = torch.tensor([[0] * (L - len(s)) + s for s in seqs], dtype=torch.float32)
            logits = _unwrap(model(Tensor(batch)))
            nxt = logits[:, -1].float().argmax(-1).tolist()
            for rid, t in zip(decode_ids, nxt):
                self._lib.lt_sched_commit(self._s, rid, int(t))
        fin = (c_int64 * cap)()
        k = self._lib.lt_sched_pop_finished(self._s, fin, cap)
        out = []
        for rid, r in self._reqs.items():
            if not r.is_finished:
                self._sync(rid)
        for i in range(k):
            r = self._reqs[int(fin[i])]
            r.is_finished = True
            r.block_ids = []
            out.append(r)
            self._retire(r.id)
        return out

    def _retire(self, rid: int) -> None:
        """A finished request leaves the books (here and in the native scheduler): a server that runs for days holds
        state for the requests in flight only.  The caller keeps the `Request` object it was handed."""
        self._lib.lt_sched_release(self._s, rid)
        self._reqs.pop(rid, None)
        try:
            self._order.remove(rid)
        except ValueError:
            pass

    def _step_kv(self, model) -> List[Request]:
        cap = max(self.max_num_seqs, 1)
        ids = (c_int64 * cap)()
        starts = (c_int32 * cap)()
        lens = (c_int32 * cap)()
        n = self._lib.lt_sched_plan(self._s, ids, starts, lens, cap)
        if n == 0:
            return []
        dec = []
        for i in range(n):
            rid, st, ln = int(ids[i]), int(starts[i]), int(lens[i])
            self._sync(rid)
            r = self._reqs[rid]
            if ln > 0:
                done = st + ln >= len(r.prompt_tokens)
                nxt = model.prefill_chunk(r.prompt_tokens[st:st + ln], st, r.block_ids, done)
                self._lib.lt_sched_commit(self._s, rid, int(nxt) if done else -1)
            else:
                dec.append((rid, st))
        if dec:
            toks = [self._tokens(rid)[pos] for rid, pos in dec]
            nxt = model.decode_batch(toks, [pos for _, pos in dec], [self._reqs[rid].block_ids for rid, _ in dec])
            for (rid, _), t in zip(dec, nxt):
                self._lib.lt_sched_commit(self._s, rid, int(t))
        fin = (c_int64 * cap)()
        k = self._lib.lt_sched_pop_finished(self._s, fin, cap)
        out = []
        for i in range(k):
            r = self._reqs[int(fin[i])]
            self._sync(r.id)
            r.is_finished = True
            r.block_ids = []
            out.append(r)
            self._retire(r.id)
        return out

    def get_block_table_tensor(self) -> Tensor:
        run = self.running_queue
        width = max([len(r.block_ids) for r in run], default=0)
        rows = [[float(b) for b in r.block_ids] + [0.0] * (width - len(r.block_ids)) for r in run]
        return Tensor(torch.tensor(rows, dtype=torch.float32).reshape(len(run), width))

    def get_context_lens_tensor(self) -> Tensor:
        return Tensor(torch.tensor([float(self._lib.lt_sched_context_len(self._s, r.id)) for r in self.running_queue],
                                   dtype=torch.float32))


# ------------------------------------------------------------------------------------------------ prefix cache
class PrefixCache:
    """Singleton map from a token prefix to its KV tensors (reference API) backed by the native token-prefix index,
    which also answers longest-prefix queries for block reuse."""

    _inst = None

    def __init__(self):
        self._lib = _h()
        self._c = self._lib.lt_prefix_create(4096)
        self._kv: Dict[tuple, list] = {}

    @staticmethod
    def get() -> "PrefixCache":
        if PrefixCache._inst is None:
            PrefixCache._inst = PrefixCache()
        return PrefixCache._inst

    def put(self, prefix: Sequence[int], kv_cache, blocks: Sequence[int] = (), *more):
        """`put(prefix, [k, v, ...])` (include/litetorch/llm_serving.h:18); the tensors may also be passed one by one,
        `put(prefix, k, v)`, as the reference's serving guide writes it.  `blocks`: KV blocks that hold the prefix."""
        key = tuple(int(t) for t in prefix)
        if isinstance(kv_cache, Tensor) or torch.is_tensor(kv_cache):
            kv_cache = [kv_cache] + ([blocks] if isinstance(blocks, Tensor) or torch.is_tensor(blocks) else []) + list(more)
            if len(kv_cache) > 1:
                blocks = ()
        self._kv[key] = list(kv_cache)
        self._lib.lt_prefix_insert(self._c, _i32(key), len(key), _i32(blocks), len(blocks))

    def get_cache(self, prefix: Sequence[int]) -> list:
        return self._kv.get(tuple(int(t) for t in prefix), [])

    def longest_prefix(self, tokens: Sequence[int], granularity: int = 1):
        """(matched length, KV blocks) of the longest cached prefix of `tokens`."""
        out = (c_int32 * 4096)()
        nb = c_int(0)
        n = self._lib.lt_prefix_lookup(self._c, _i32(tokens), len(tokens), granularity, out, 4096, ctypes.byref(nb))
        return n, [int(out[i]) for i in range(min(nb.value, 4096))]

    def clear(self):
        self._kv.clear()
        self._lib.lt_prefix_destroy(self._c)
        self._c = self._lib.lt_prefix_create(4096)


# ------------------------------------------------------------------------------------------------ speculative / Medusa
def _greedy_last(model, tokens: List[int]):
    logits = _unwrap(model(Tensor(torch.tensor([tokens], dtype=torch.float32))))
    return logits[0].float()


class SpeculativeEngine:
    """Greedy draft-k / verify (src/nn/llm_serving.cpp:42-139): the draft proposes `lookahead` tokens, one target
    forward scores them all, the longest agreeing prefix is accepted and the target's own next token is appended."""

    def __init__(self, draft_model, target_model):
        self.draft_model, self.target_model = draft_model, target_model

    def generate(self, prompt: Sequence[int], max_new_tokens: int, lookahead: int = 4) -> List[int]:
        result = [int(t) for t in prompt]
        generated = 0
        while generated < max_new_tokens:
            cur = list(result)
            draft = []
            for _ in range(lookahead):
                t = int(_greedy_last(self.draft_model, cur)[-1].argmax().item())
                draft.append(t)
                cur.append(t)
            tl = _greedy_last(self.target_model, cur)
            base = len(result)
            accept = 0
            for k in range(lookahead):
                if int(tl[base - 1 + k].argmax().item()) == draft[k]:
                    accept += 1
                else:
                    break
            for a in range(accept):
                if generated >= max_new_tokens:
                    break
                result.append(draft[a])
                generated += 1
            if generated >= max_new_tokens:
                break
            result.append(int(tl[base - 1 + accept].argmax().item()))
            generated += 1
        return result


class MedusaHead:
    """Extra LM head applied to the base model's logits of the last position (src/llm/medusa.cpp:10-36)."""

    def __init__(self, in_features: int, vocab_size: int):
        scale = 1.0 / (in_features ** 0.5)
        self.weight = Tensor(((torch.rand(vocab_size, in_features) * 2 - 1) * scale).requires_grad_(True))
        self.bias = Tensor(torch.zeros(vocab_size).requires_grad_(True))
        self.training = True

    def forward(self, x: Tensor) -> Tensor:
        return Tensor(torch.nn.functional.linear(_unwrap(x), _unwrap(self.weight), _unwrap(self.bias)))

    __call__ = forward

    def parameters(self):
        return [self.weight, self.bias]

    def to(self, device):
        from .core import _as_device
        d = _as_device(device)
        self.weight = Tensor(_unwrap(self.weight).detach().to(d).requires_grad_(True))
        self.bias = Tensor(_unwrap(self.bias).detach().to(d).requires_grad_(True))
        return self


class MedusaEngine:
    """Base model + Medusa heads: head i guesses the token i+1 steps ahead; a second base forward over the
    candidate continuation verifies the guesses greedily (src/llm/medusa.cpp:38-124)."""

    def __init__(self, base_model, medusa_heads: Sequence[MedusaHead]):
        self.base_model, self.medusa_heads = base_model, list(medusa_heads)

    def generate(self, prompt: Sequence[int], max_new_tokens: int, lookahead: int = 2) -> List[int]:
        tokens = [int(t) for t in prompt]
        n0 = len(tokens)
        while len(tokens) - n0 < max_new_tokens:
            logits = _greedy_last(self.base_model, tokens)
            last = logits[-1]
            nxt = int(last.argmax().item())
            cand = [nxt]
            for head in self.medusa_heads[:lookahead]:
                cand.append(int(_unwrap(head.forward(Tensor(last[None])))[0].argmax().item()))
            ver = _greedy_last(self.base_model, tokens + cand)
            accepted = [nxt]
            for i in range(1, len(cand)):
                if int(ver[len(tokens) - 1 + i].argmax().item()) == cand[i]:
                    accepted.append(cand[i])
                else:
                    break
            for t in accepted:
                if len(tokens) - n0 >= max_new_tokens:
                    break
                tokens.append(t)
        return tokens


class GuidedDecoder:
    """Masks logits so that `prefix + token` stays compatible with "digits", "prefix:<s>" or "regex:<re>"."""

    def __init__(self, vocabulary: Sequence[str]):
        self.vocab = list(vocabulary)
        enc = [v.encode("utf-8") for v in self.vocab]
        self._blob = b"".join(enc)
        offs = [0]
        for e in enc:
            offs.append(offs[-1] + len(e))
        self._offs = (c_int64 * len(offs))(*offs)

    def allowed(self, prefix: str, target_pattern: str) -> torch.Tensor:
        V = len(self.vocab)
        out = (c_uint8 * V)()
        _h().lt_guided_mask(target_pattern.encode(), prefix.encode(), self._blob, self._offs, V, out)
        return torch.tensor(list(out), dtype=torch.bool)

    def apply_mask(self, logits: Tensor, prefix: str, target_pattern: str) -> None:
        t = _unwrap(logits)
        V = min(t.shape[-1], len(self.vocab))
        ok = self.allowed(prefix, target_pattern)[:V].to(t.device)
        with torch.no_grad():
            t[..., :V].masked_fill_(~ok, -1e9)
