"""Llama-style decoder (RMSNorm, RoPE, GQA attention, SwiGLU) as an explicit forward/backward engine.

The training hot path does not go through autograd: every layer has a hand-written backward that calls
the sm_100a kernels directly (tcgen05 GEMMs in the three operand layouts, FlashAttention fwd/bwd, fused
residual+RMSNorm, RoPE in place on the fused QKV buffer, SwiGLU, in-place cross-entropy gradient,
flat-buffer AdamW).  Weights live in flat buffers described by `ParamSpec`s so that the optimizer is one
launch and so that the ZeRO-3 engine (`litetorch_b200.parallel.fsdp`) can shard them by rows.

The reference builds its decoder from `lt.nn.TransformerDecoderLayer` (post-LN, GELU, LayerNorm:
src/nn/transformer.cpp:7-70) on the autograd tape; RMSNorm/SwiGLU/causal GQA attention are claimed in its
README (README.md:23-25) but absent from its sources, so this model implements the claimed capability.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field, asdict
from typing import Dict, List, Optional, Tuple

import torch

from ..ops import kernels as K
from ..ops import kernels_ref as K_ref


def kernels_for(device):
    """The kernel front-end for tensors on `device`: the sm_100a library on CUDA, its PyTorch twin on the CPU."""
    return K if torch.device(device).type == "cuda" else K_ref


class SingleTPMixin:
    """Weight-provider methods of the tensor-parallel schedule for providers that hold whole matrices (tp = 1):
    a column-parallel linear is a plain GEMM that hands back its own input as the "gathered" activation, a
    row-parallel linear is a plain GEMM with the residual in the epilogue."""
    tp = 1
    tp_rank = 0
    vocab_start = 0

    def col_linear(self, x, name):
        return self.linear(x, name), x

    def row_linear(self, x, name, residual=None):
        return self.linear(x, name, residual=residual)

    def col_dgrad(self, dy, name):
        return self.dgrad(dy, name)

    def row_dgrad(self, dy, name):
        return self.dgrad(dy, name), dy

    def reduce_ce_stats(self, stats):
        return stats

    def gather_slot(self, rows, cols):
        """Where the producer of the next gathered activation should write it (None: anywhere)."""
        return None


@dataclass
class LlamaConfig:
    vocab_size: int = 32000
    n_layers: int = 22
    d_model: int = 2048
    n_heads: int = 32
    n_kv_heads: int = 4
    head_dim: int = 64
    ffn: int = 5632
    rms_eps: float = 1e-5
    rope_theta: float = 1e4
    max_seq: int = 2048
    init_std: float = 0.02
    name: str = "llama-1.1b"

    @property
    def qkv_dim(self) -> int:
        return (self.n_heads + 2 * self.n_kv_heads) * self.head_dim

    def num_params(self) -> int:
        per_layer = (self.qkv_dim * self.d_model + self.d_model * self.n_heads * self.head_dim +
                     3 * self.ffn * self.d_model + 2 * self.d_model)
        return self.n_layers * per_layer + 2 * self.vocab_size * self.d_model + self.d_model

    def flops_per_token(self, seq_len: int) -> float:
        """Training FLOPs per token (fwd + bwd = 3x forward), causal attention counted at half."""
        mm = self.n_layers * (self.qkv_dim * self.d_model + self.d_model * self.n_heads * self.head_dim +
                              3 * self.ffn * self.d_model) + self.vocab_size * self.d_model
        attn = self.n_layers * 6.0 * seq_len * self.n_heads * self.head_dim  # 3 x (QK^T + PV), causal half
        return 6.0 * mm + attn

    # ---- presets named by the benchmark configurations
    @staticmethod
    def tiny(**kw) -> "LlamaConfig":
        return LlamaConfig(vocab_size=512, n_layers=2, d_model=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn=512,
                           max_seq=256, name="llama-tiny", **kw)

    @staticmethod
    def llama_1b(**kw) -> "LlamaConfig":
        return LlamaConfig(**kw)

    @staticmethod
    def llama_3b(**kw) -> "LlamaConfig":
        return LlamaConfig(vocab_size=32000, n_layers=28, d_model=3072, n_heads=24, n_kv_heads=8, head_dim=128,
                           ffn=8192, rope_theta=1e4, max_seq=32768, name="llama-3b", **kw)

    @staticmethod
    def llama3_8b(**kw) -> "LlamaConfig":
        return LlamaConfig(vocab_size=128256, n_layers=32, d_model=4096, n_heads=32, n_kv_heads=8, head_dim=128,
                           ffn=14336, rope_theta=5e5, max_seq=8192, name="llama3-8b", **kw)


@dataclass
class ParamSpec:
    name: str
    shape: Tuple[int, ...]
    kind: str            # "matrix" (row-shardable, weight decay) or "vector" (norm gains: replicated, no decay)
    offset: int = 0      # element offset in the flat buffer of its kind


def param_specs(cfg: LlamaConfig) -> List[ParamSpec]:
    """Every parameter in `parameters()` order: embedding, per layer (attn_norm, wqkv, wo, mlp_norm, w_gu, w_down),
    final norm, lm_head."""
    specs = [ParamSpec("embed", (cfg.vocab_size, cfg.d_model), "matrix")]
    for i in range(cfg.n_layers):
        p = "layers.%d." % i
        specs += [
            ParamSpec(p + "attn_norm", (cfg.d_model,), "vector"),
            ParamSpec(p + "wqkv", (cfg.qkv_dim, cfg.d_model), "matrix"),
            ParamSpec(p + "wo", (cfg.d_model, cfg.n_heads * cfg.head_dim), "matrix"),
            ParamSpec(p + "mlp_norm", (cfg.d_model,), "vector"),
            ParamSpec(p + "w_gu", (2 * cfg.ffn, cfg.d_model), "matrix"),
            ParamSpec(p + "w_down", (cfg.d_model, cfg.ffn), "matrix"),
        ]
    specs += [ParamSpec("final_norm", (cfg.d_model,), "vector"),
              ParamSpec("lm_head", (cfg.vocab_size, cfg.d_model), "matrix")]
    off = {"matrix": 0, "vector": 0}
    for s in specs:
        s.offset = off[s.kind]
        n = 1
        for d in s.shape:
            n *= d
        off[s.kind] += (n + 127) // 128 * 128
    return specs


def rope_tables(cfg: LlamaConfig, device, max_seq: Optional[int] = None):
    T = max_seq or cfg.max_seq
    inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, cfg.head_dim, 2, device=device, dtype=torch.float64) / cfg.head_dim))
    ang = torch.arange(T, device=device, dtype=torch.float64)[:, None] * inv[None, :]
    return ang.cos().float().contiguous(), ang.sin().float().contiguous()


class LocalWeights(SingleTPMixin):
    """All parameters resident on one GPU: flat bf16 parameters + flat bf16 gradients + fp32 master/m/v."""

    def __init__(self, cfg: LlamaConfig, device, seed: int = 0, param_dtype=torch.bfloat16):
        self.cfg = cfg
        self.K = kernels_for(device)
        self.specs = param_specs(cfg)
        self.by_name = {s.name: s for s in self.specs}
        sizes = {"matrix": 0, "vector": 0}
        for s in self.specs:
            sizes[s.kind] = max(sizes[s.kind], s.offset + (math.prod(s.shape) + 127) // 128 * 128)
        self.n_matrix, self.n_vector = sizes["matrix"], sizes["vector"]
        n = self.n_matrix + self.n_vector
        self.flat_p = torch.zeros(n, dtype=param_dtype, device=device)
        self.flat_g = torch.zeros(n, dtype=param_dtype, device=device)
        self.master = torch.zeros(n, dtype=torch.float32, device=device)
        self.m = torch.zeros(n, dtype=torch.float32, device=device)
        self.v = torch.zeros(n, dtype=torch.float32, device=device)
        gen = torch.Generator(device=device).manual_seed(seed)
        for s in self.specs:
            w = self.master_view(s.name)
            if s.kind == "matrix":
                w.normal_(0.0, cfg.init_std, generator=gen)
            else:
                w.fill_(1.0)
        self.flat_p.copy_(self.master)

    def _base(self, s: ParamSpec) -> int:
        return s.offset if s.kind == "matrix" else self.n_matrix + s.offset

    def _view(self, flat, name):
        s = self.by_name[name]
        b = self._base(s)
        return flat[b:b + math.prod(s.shape)].view(*s.shape)

    def p(self, name) -> torch.Tensor:
        return self._view(self.flat_p, name)

    def g(self, name) -> torch.Tensor:
        return self._view(self.flat_g, name)

    def master_view(self, name) -> torch.Tensor:
        return self._view(self.master, name)

    # ---- GEMM providers (the ZeRO-3 weights object overrides these with fused all-gather variants)
    def linear(self, x, name, **kw):
        return self.K.gemm(x, self.p(name), **kw)

    def dgrad(self, dy, name, **kw):
        return self.K.gemm(dy, self.p(name), b_major=1, **kw)

    def wgrad(self, dy, x, name, accumulate=False):
        return self.K.gemm(dy, x, a_major=1, b_major=1, out=self.g(name), accumulate=accumulate)

    def vector_grad(self, name):
        return self.g(name)

    def zero_grad_embed(self):
        self.g("embed").zero_()

    def embedding(self, tokens):
        return self.K.embedding_fwd(tokens, self.p("embed"))

    def embedding_backward(self, tokens, dx):
        self.K.embedding_bwd(tokens, dx, self.g("embed"))

    def optimizer_step(self, *, lr, beta1, beta2, eps, weight_decay, step, dyn=None):
        nm = self.n_matrix
        if getattr(self, "_hyper", None) is not None and getattr(self, "_updated", 0) == nm and dyn is None:
            # every matrix was updated bucket by bucket on the side stream during the backward pass
            self.K.adam_flat(self.master[nm:], self.flat_g[nm:], self.m[nm:], self.v[nm:], self.flat_p[nm:], lr=lr, beta1=beta1,
                        beta2=beta2, eps=eps, wd=0.0, step=step, adamw=True)
            torch.cuda.current_stream().wait_stream(self._side)
            self._updated = 0
            return
        if getattr(self, "_updated", 0):
            raise RuntimeError("optimizer_step after a partial overlapped update")
        self.K.adam_flat(self.master[:nm], self.flat_g[:nm], self.m[:nm], self.v[:nm], self.flat_p[:nm], lr=lr, beta1=beta1,
                    beta2=beta2, eps=eps, wd=weight_decay, step=step, adamw=True, dyn=dyn)
        self.K.adam_flat(self.master[nm:], self.flat_g[nm:], self.m[nm:], self.v[nm:], self.flat_p[nm:], lr=lr, beta1=beta1,
                    beta2=beta2, eps=eps, wd=0.0, step=step, adamw=True, dyn=dyn)

    # ---- AdamW overlapped with the backward pass: as soon as the weight gradients of a bucket ("head", a layer, "embed")
    # have been issued, its slice of the flat buffers is updated on a side stream.  The update is bound by HBM
    # bandwidth and the GEMMs it runs beside are bound by the tensor cores, so most of it is hidden; the vectors
    # (norm gains) and whatever was not covered are updated at the end.
    def _bucket_range(self, bucket):
        if bucket == "embed":
            names = ["embed"]
        elif bucket == "head":
            names = ["lm_head"]
        else:
            names = ["layers.%d.%s" % (bucket, n) for n in ("wqkv", "wo", "w_gu", "w_down")]
        lo = min(self.by_name[n].offset for n in names)
        hi = max(self.by_name[n].offset + (math.prod(self.by_name[n].shape) + 127) // 128 * 128 for n in names)
        return lo, hi

    def begin_step(self, **hyper):
        self._hyper = hyper
        self._updated = 0
        if getattr(self, "_side", None) is None and self.flat_p.is_cuda:
            self._side = torch.cuda.Stream(device=self.flat_p.device)

    def bucket_done(self, bucket):
        """Hook: all weight gradients of a bucket ("head", layer index, "embed") have been issued."""
        h = getattr(self, "_hyper", None)
        if h is None or getattr(self, "_side", None) is None:
            return
        a, b = self._bucket_range(bucket)
        self._side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self._side):
            self.K.adam_flat(self.master[a:b], self.flat_g[a:b], self.m[a:b], self.v[a:b], self.flat_p[a:b], lr=h["lr"],
                        beta1=h["beta1"], beta2=h["beta2"], eps=h["eps"], wd=h["weight_decay"], step=h["step"], adamw=True)
        self._updated += b - a

    def finish_step(self):
        self._hyper = None

    def parameters(self) -> List[torch.Tensor]:
        return [self.master_view(s.name) for s in self.specs]

    def state_tensors(self) -> Dict[str, torch.Tensor]:
        """Everything a restart needs besides the step count: fp32 masters and AdamW moments (flat buffers)."""
        return {"master": self.master, "m": self.m, "v": self.v}

    def after_load(self) -> None:
        self.flat_p.copy_(self.master)

    def load_parameters(self, tensors: List[torch.Tensor]):
        for s, t in zip(self.specs, tensors):
            self.master_view(s.name).copy_(t.to(self.master.device, torch.float32).view(*s.shape))
        self.flat_p.copy_(self.master)


class LlamaEngine:
    """Forward + backward + optimizer step of a Llama-style decoder on the sm_100a kernels.

    The schedule is written once for tensor parallelism with sequence parallelism and degenerates to the plain
    single-GPU schedule when the weight provider has `tp == 1`: the residual stream, the norms and their
    gradients live on this rank's block of M / tp token rows; a column-parallel linear (QKV, gate/up, LM head)
    gathers its input over the tensor-parallel group and produces this rank's heads / feed-forward columns /
    vocabulary slice for all M rows; a row-parallel linear (attention output, down projection) reduces its
    partial products over the group and scatters the rows back (`col_linear`, `row_linear`, `col_dgrad`,
    `row_dgrad` of the provider - fused all-gather -> GEMM and GEMM -> reduce-scatter kernels in
    `parallel.hybrid.HybridWeights`).  Every rank of a tensor-parallel group is given the same [B, T] batch.
    Counterparts in the reference: ColumnParallelLinear / RowParallelLinear (src/nn/parallel_linear.cpp:31-106)
    inside an FSDP-wrapped module (src/distributed/fsdp_wrapper.cpp:106-156).
    """

    def __init__(self, cfg: LlamaConfig, device="cuda", weights=None, seed: int = 0, lr: float = 3e-4,
                 betas=(0.9, 0.95), eps: float = 1e-8, weight_decay: float = 0.1, activation_checkpointing: bool = False,
                 world_size: int = 1, head_chunk_rows: int = 0, grad_clip: float = 0.0):
        self.cfg = cfg
        # > 0: the gradient is scaled so that its global L2 norm does not exceed this value (the reference's
        # Ops::clip_grad_norm_, src/ops/clip_grad.cpp); a non-finite gradient skips the update
        self.grad_clip = float(grad_clip)
        self.last_grad_norm = None            # device scalar: norm before clipping, of the latest clipped step
        # > 0: the LM head and the loss go through in chunks of that many token rows, so that only [chunk, vocab]
        # logits exist at a time (whole weights on this rank only)
        self.head_chunk_rows = int(head_chunk_rows)
        self.device = torch.device(device)
        self.K = kernels_for(self.device)
        self.w = weights if weights is not None else LocalWeights(cfg, self.device, seed)
        self.lr, self.betas, self.eps, self.weight_decay = lr, betas, eps, weight_decay
        if self.grad_clip > 0 and not isinstance(self.w, LocalWeights):
            raise NotImplementedError("gradient clipping needs the whole gradient before the first update: it is "
                                      "available with unsharded weights; the sharded providers update each bucket "
                                      "under the backward pass")
        # True: every layer is recomputed in the backward pass; an integer k: only the first k layers are
        self.ckpt_layers = cfg.n_layers if activation_checkpointing is True else int(activation_checkpointing or 0)
        self.ckpt = self.ckpt_layers > 0
        self.world_size = world_size          # data-parallel replicas the gradient is averaged over
        self.step_count = 0
        self.cos, self.sin = rope_tables(cfg, self.device)
        self.kernel_launches = 0
        tp = self.w.tp
        assert cfg.n_heads % tp == 0 and cfg.n_kv_heads % tp == 0 and cfg.ffn % tp == 0 and cfg.vocab_size % tp == 0, \
            "heads, kv heads, ffn and vocabulary must divide over the tensor-parallel group"
        self.Hq, self.Hkv = cfg.n_heads // tp, cfg.n_kv_heads // tp
        self.qkv_local = (self.Hq + 2 * self.Hkv) * cfg.head_dim

    # ------------------------------------------------------------------------------------------ layer
    def _layer_fwd(self, i: int, x: torch.Tensor, B: int, T: int):
        cfg, w, K = self.cfg, self.w, self.K
        p = "layers.%d." % i
        Hq, Hkv, hd = self.Hq, self.Hkv, cfg.head_dim
        h1, _, _, rstd1 = K.norm_fwd(x, w.p(p + "attn_norm"), eps=cfg.rms_eps, out=w.gather_slot(*x.shape))
        qkv, h1f = w.col_linear(h1, p + "wqkv")
        K.rope_(qkv, self.cos, self.sin, T, Hq, hd, col_offset=0)
        K.rope_(qkv, self.cos, self.sin, T, Hkv, hd, col_offset=Hq * hd)
        q, k, v = self._split_qkv(qkv, B, T)
        o, lse = K.flash_fwd(q, k, v, causal=True)
        o2 = o.view(B * T, Hq * hd)
        x1 = w.row_linear(o2, p + "wo", residual=x)
        h2, _, _, rstd2 = K.norm_fwd(x1, w.p(p + "mlp_norm"), eps=cfg.rms_eps, out=w.gather_slot(*x1.shape))
        gu, h2f = w.col_linear(h2, p + "w_gu")
        hm = K.swiglu_fwd(gu)
        x2 = w.row_linear(hm, p + "w_down", residual=x1)
        self.kernel_launches += 11
        return x2, (x, h1f, rstd1, qkv, o, lse, x1, h2f, rstd2, gu, hm)

    def _split_qkv(self, qkv, B, T):
        Hq, Hkv, hd = self.Hq, self.Hkv, self.cfg.head_dim
        q3 = qkv.view(B, T, self.qkv_local)
        q = q3[:, :, :Hq * hd].view(B, T, Hq, hd)
        k = q3[:, :, Hq * hd:(Hq + Hkv) * hd].view(B, T, Hkv, hd)
        v = q3[:, :, (Hq + Hkv) * hd:].view(B, T, Hkv, hd)
        return q, k, v

    def _layer_bwd(self, i: int, dx2: torch.Tensor, ctx, B: int, T: int, accumulate: bool):
        cfg, w, K = self.cfg, self.w, self.K
        p = "layers.%d." % i
        Hq, Hkv, hd = self.Hq, self.Hkv, cfg.head_dim
        x, h1f, rstd1, qkv, o, lse, x1, h2f, rstd2, gu, hm = ctx
        # MLP
        dhm, dx2f = w.row_dgrad(dx2, p + "w_down")
        w.wgrad(dx2f, hm, p + "w_down", accumulate)
        dgu = K.swiglu_bwd(gu, dhm, inplace=True)
        dh2 = w.col_dgrad(dgu, p + "w_gu")
        w.wgrad(dgu, h2f, p + "w_gu", accumulate)
        dx1, _, _ = K.norm_bwd(dh2, x1, w.p(p + "mlp_norm"), None, rstd2, dres=dx2, dw=w.vector_grad(p + "mlp_norm"),
                               accumulate=accumulate, out=w.gather_slot(*x1.shape))
        # attention
        o2 = o.view(B * T, Hq * hd)
        do, dx1f = w.row_dgrad(dx1, p + "wo")
        w.wgrad(dx1f, o2, p + "wo", accumulate)
        dqkv = torch.empty_like(qkv)
        q, k, v = self._split_qkv(qkv, B, T)
        dq, dk, dv = self._split_qkv(dqkv, B, T)
        K.flash_bwd(q, k, v, o, lse, do.view(B, T, Hq, hd), causal=True, dq=dq, dk=dk, dv=dv)
        K.rope_(dqkv, self.cos, self.sin, T, Hq, hd, col_offset=0, backward=True)
        K.rope_(dqkv, self.cos, self.sin, T, Hkv, hd, col_offset=Hq * hd, backward=True)
        dh1 = w.col_dgrad(dqkv, p + "wqkv")
        w.wgrad(dqkv, h1f, p + "wqkv", accumulate)
        # The gradient that leaves this layer is the input of the next gathered GEMM - unless that layer recomputes its
        # forward pass first (its gathers would take the slot), or there is no next layer (embedding).
        direct = i > 0 and (i - 1) >= self.ckpt_layers
        dx, _, _ = K.norm_bwd(dh1, x, w.p(p + "attn_norm"), None, rstd1, dres=dx1, dw=w.vector_grad(p + "attn_norm"),
                              accumulate=accumulate, out=w.gather_slot(*x.shape) if direct else None)
        self.kernel_launches += 22
        return dx

    # ------------------------------------------------------------------------------------------ model
    def forward_backward(self, tokens: torch.Tensor, targets: torch.Tensor, *, accumulate: bool = False,
                         loss_scale: float = 1.0, fused_update: bool = False) -> torch.Tensor:
        """One micro-batch: returns the mean token loss (device scalar); gradients are left in the flat buffer.

        fused_update: sharded weights may reduce and apply each bucket's gradients as soon as its backward is done
        (only valid for the last micro-batch of a step, after `begin_step`)."""
        cfg, w, K = self.cfg, self.w, self.K
        B, T = tokens.shape
        M = B * T
        tok = tokens.reshape(-1)
        tgt = targets.reshape(-1)
        x = w.embedding(tok)
        saved = []
        for i in range(cfg.n_layers):
            if i < self.ckpt_layers:
                saved.append(x)
                x, _ = self._layer_fwd(i, x, B, T)
            else:
                x, ctx = self._layer_fwd(i, x, B, T)
                saved.append(ctx)
        hf, _, _, rstd_f = K.norm_fwd(x, w.p("final_norm"), eps=cfg.rms_eps, out=w.gather_slot(*x.shape))
        if self.head_chunk_rows > 0 and isinstance(w, LocalWeights):
            # chunked head: logits of one chunk -> their gradient in place -> the two gradient GEMMs; no [M, V] tensor
            dhf = torch.empty_like(hf)
            loss = torch.zeros((), dtype=torch.float32, device=hf.device)
            for ci, s0 in enumerate(range(0, M, self.head_chunk_rows)):
                hc, tc = hf[s0:s0 + self.head_chunk_rows], tgt[s0:s0 + self.head_chunk_rows]
                lg = w.linear(hc, "lm_head")
                rows = K.ce_finish(lg, tc, K.ce_stats(lg, tc), grad_scale=loss_scale / (M * self.world_size))
                loss = loss + rows.sum()
                K.gemm(lg, w.p("lm_head"), b_major=1, out=dhf[s0:s0 + self.head_chunk_rows])
                w.wgrad(lg, hc, "lm_head", accumulate or ci > 0)
            loss = loss / M
        else:
            logits, hff = w.col_linear(hf, "lm_head")
            stats = w.reduce_ce_stats(K.ce_stats(logits, tgt, w.vocab_start))
            rows = K.ce_finish(logits, tgt, stats, vocab_start=w.vocab_start, grad_scale=loss_scale / (M * self.world_size))
            loss = rows.sum() / M
            dhf = w.col_dgrad(logits, "lm_head")
            w.wgrad(logits, hff, "lm_head", accumulate)
            del logits, hff
        if fused_update:
            w.bucket_done("head")
        dx, _, _ = K.norm_bwd(dhf, x, w.p("final_norm"), None, rstd_f, dw=w.vector_grad("final_norm"), accumulate=accumulate,
                              out=w.gather_slot(*x.shape) if cfg.n_layers - 1 >= self.ckpt_layers else None)
        for i in reversed(range(cfg.n_layers)):
            if i < self.ckpt_layers:
                _, ctx = self._layer_fwd(i, saved[i], B, T)
            else:
                ctx = saved[i]
            dx = self._layer_bwd(i, dx, ctx, B, T, accumulate)
            if fused_update:
                w.bucket_done(i)
            saved[i] = None
        if not accumulate:
            w.zero_grad_embed()
        w.embedding_backward(tok, dx)
        if fused_update:
            w.bucket_done("embed")
        self.kernel_launches += 12
        return loss

    def forward_logits(self, tokens: torch.Tensor) -> torch.Tensor:
        """Logits of this rank's vocabulary slice for every token ([B, T, vocab / tp])."""
        cfg, w, K = self.cfg, self.w, self.K
        B, T = tokens.shape
        x = w.embedding(tokens.reshape(-1))
        for i in range(cfg.n_layers):
            x, _ = self._layer_fwd(i, x, B, T)
        hf, _, _, _ = K.norm_fwd(x, w.p("final_norm"), eps=cfg.rms_eps)
        return w.col_linear(hf, "lm_head")[0].view(B, T, cfg.vocab_size // w.tp)

    def eval_loss(self, tokens: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        """Mean token loss of a batch (device scalar) from a forward pass only: gradients, moments and the step count are
        left alone (validation between training steps).  Under tensor parallelism the loss is reduced over the group's
        vocabulary slices; under data parallelism it is the loss of this rank's batch."""
        w, K = self.w, self.K
        B, T = tokens.shape
        logits = self.forward_logits(tokens).view(B * T, -1)
        tgt = targets.reshape(-1)
        stats = w.reduce_ce_stats(K.ce_stats(logits, tgt, w.vocab_start))
        rows = K.ce_finish(logits, tgt, stats, vocab_start=w.vocab_start, write_grad=False)
        self.kernel_launches += 2
        return rows.sum() / (B * T)

    def optimizer_step(self, dyn=None):
        self.step_count += 1
        self.w.optimizer_step(lr=self.lr, beta1=self.betas[0], beta2=self.betas[1], eps=self.eps,
                              weight_decay=self.weight_decay, step=self.step_count, dyn=dyn)
        self.kernel_launches += 2

    def _clip_dyn(self) -> torch.Tensor:
        """{gradient multiplier, non-finite flag, norm} on the device from one pass over the flat gradient: the AdamW
        kernel multiplies every gradient by the first and returns at once when the second is set (no host sync)."""
        stats = torch.zeros(2, dtype=torch.float32, device=self.device)
        dyn = torch.zeros(3, dtype=torch.float32, device=self.device)
        self.K.sumsq(self.w.flat_g, stats)
        self.K.clip_coef(stats, dyn, self.grad_clip)
        self.last_grad_norm = dyn[2]
        self.kernel_launches += 2
        return dyn

    def train_step(self, tokens: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        """The public one-call training step: forward, backward, AdamW.  Returns the loss (device scalar)."""
        if self.grad_clip > 0:
            loss = self.forward_backward(tokens, targets)
            self.optimizer_step(dyn=self._clip_dyn())
            return loss
        self.w.begin_step(lr=self.lr, beta1=self.betas[0], beta2=self.betas[1], eps=self.eps,
                          weight_decay=self.weight_decay, step=self.step_count + 1)
        loss = self.forward_backward(tokens, targets, fused_update=True)
        self.optimizer_step()
        self.w.finish_step()
        return loss


    def train_step_accumulated(self, micro_batches) -> torch.Tensor:
        """One optimizer step over several micro-batches (gradient accumulation): `micro_batches` is a sequence of
        (tokens, targets) pairs of equal size; every micro-batch's gradient is scaled by 1 / k and added into the flat
        gradient buffer, the sharded reduce + AdamW of each bucket runs under the LAST micro-batch's backward pass.
        Returns the mean loss (device scalar).  Equal to `train_step` on the concatenated batch up to rounding."""
        k = len(micro_batches)
        if k == 1:
            return self.train_step(*micro_batches[0])
        if self.grad_clip > 0:
            total = None
            for i, (tok, tgt) in enumerate(micro_batches):
                loss = self.forward_backward(tok, tgt, accumulate=i > 0, loss_scale=1.0 / k)
                total = loss / k if total is None else total + loss / k
            self.optimizer_step(dyn=self._clip_dyn())
            return total
        self.w.begin_step(lr=self.lr, beta1=self.betas[0], beta2=self.betas[1], eps=self.eps,
                          weight_decay=self.weight_decay, step=self.step_count + 1)
        total = None
        for i, (tok, tgt) in enumerate(micro_batches):
            loss = self.forward_backward(tok, tgt, accumulate=i > 0, loss_scale=1.0 / k, fused_update=(i == k - 1))
            total = loss / k if total is None else total + loss / k
        self.optimizer_step()
        self.w.finish_step()
        return total


class TorchLlama(torch.nn.Module):
    """The same architecture in stock PyTorch (fp32 or bf16): oracle for the tests and the cuBLAS/SDPA baseline."""

    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.cfg = cfg
        nn = torch.nn
        self.embed = nn.Parameter(torch.empty(cfg.vocab_size, cfg.d_model))
        self.layers = nn.ParameterList()
        self.names = []
        for s in param_specs(cfg):
            self.names.append(s.name)
        self.params = nn.ParameterDict({s.name.replace(".", "_"): nn.Parameter(torch.empty(*s.shape)) for s in param_specs(cfg)})
        del self.embed, self.layers

    def P(self, name):
        return self.params[name.replace(".", "_")]

    def load_from(self, tensors):
        with torch.no_grad():
            for s, t in zip(param_specs(self.cfg), tensors):
                self.P(s.name).copy_(t.view(*s.shape))

    @staticmethod
    def _rope(x, cos, sin):
        # x: [B, T, H, D], interleaved pairs
        c = cos[None, :x.shape[1], None, :].to(x.dtype)
        s = sin[None, :x.shape[1], None, :].to(x.dtype)
        x0, x1 = x[..., 0::2], x[..., 1::2]
        return torch.stack([x0 * c - x1 * s, x0 * s + x1 * c], dim=-1).flatten(-2)

    def _norm(self, x, w):
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.cfg.rms_eps)).to(x.dtype) * w

    def forward(self, tokens):
        cfg = self.cfg
        B, T = tokens.shape
        Hq, Hkv, hd = cfg.n_heads, cfg.n_kv_heads, cfg.head_dim
        cos, sin = rope_tables(cfg, tokens.device, T)
        x = self.P("embed")[tokens]
        for i in range(cfg.n_layers):
            p = "layers.%d." % i
            h = self._norm(x, self.P(p + "attn_norm"))
            qkv = h @ self.P(p + "wqkv").t()
            q = qkv[..., :Hq * hd].view(B, T, Hq, hd)
            k = qkv[..., Hq * hd:(Hq + Hkv) * hd].view(B, T, Hkv, hd)
            v = qkv[..., (Hq + Hkv) * hd:].view(B, T, Hkv, hd)
            q, k = self._rope(q, cos, sin), self._rope(k, cos, sin)
            o = torch.nn.functional.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                                                 is_causal=True, enable_gqa=True)
            x = x + o.transpose(1, 2).reshape(B, T, Hq * hd) @ self.P(p + "wo").t()
            h = self._norm(x, self.P(p + "mlp_norm"))
            gu = h @ self.P(p + "w_gu").t()
            x = x + (torch.nn.functional.silu(gu[..., :cfg.ffn]) * gu[..., cfg.ffn:]) @ self.P(p + "w_down").t()
        return self._norm(x, self.P("final_norm")) @ self.P("lm_head").t()
