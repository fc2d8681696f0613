"""`lt.nn`: modules of the reference API (src/bindings/python_bindings.cpp:318-584) on torch tensors and the
sm_100a kernels.

`Module` keeps the reference contract (include/litetorch/nn.h:13-49): `forward`, `parameters()` in a fixed
order (checkpoints are positional), `to`, `train/eval`, `children`, forward pre/post hooks, `compile`.
Layers added because the Llama-style configurations need them and the reference only claims them:
`RMSNorm`, `SiLU`, `SwiGLU`, `LlamaMLP`, `GQAttention`.
"""
from __future__ import annotations

import math
from typing import Callable, List, Optional, Sequence

import torch

from ..core import DataType, Device, Tensor, _as_device, _unwrap
from ..ops import Ops
from ..ops import functional as Fn


class Module:
    def __init__(self):
        object.__setattr__(self, "training", True)
        object.__setattr__(self, "_fwd_pre_hooks", [])
        object.__setattr__(self, "_fwd_hooks", [])
        object.__setattr__(self, "_compiled", False)

    # ---- structure
    def forward(self, x):
        raise NotImplementedError

    def _own_tensors(self):
        for k, v in vars(self).items():
            if isinstance(v, Tensor) and _unwrap(v).requires_grad:
                yield k, v

    def children(self) -> List["Module"]:
        out = []
        for v in vars(self).values():
            if isinstance(v, Module):
                out.append(v)
            elif isinstance(v, (list, tuple)):
                out += [m for m in v if isinstance(m, Module)]
        return out

    def parameters(self) -> List[Tensor]:
        ps = [v for _, v in self._own_tensors()]
        for c in self.children():
            ps += c.parameters()
        return ps

    def to(self, device) -> "Module":
        dev = _as_device(device)
        for k, v in list(vars(self).items()):
            if isinstance(v, Tensor):
                t = _unwrap(v)
                nt = t.detach().to(dev)
                if t.requires_grad:
                    nt.requires_grad_(True)
                setattr(self, k, Tensor(nt, v._dtype_tag))
        for c in self.children():
            c.to(device)
        return self

    def cast(self, dtype: DataType) -> "Module":
        """Convert floating-point parameters (bf16 training keeps fp32 masters in the optimizer)."""
        from ..core import _TO_TORCH
        td = _TO_TORCH[dtype]
        for k, v in list(vars(self).items()):
            if isinstance(v, Tensor) and _unwrap(v).is_floating_point():
                t = _unwrap(v)
                nt = t.detach().to(td)
                if t.requires_grad:
                    nt.requires_grad_(True)
                setattr(self, k, Tensor(nt))
        for c in self.children():
            c.cast(dtype)
        return self

    def train(self, mode: bool = True):
        self.training = mode
        for c in self.children():
            c.train(mode)
        return self

    def eval(self):
        return self.train(False)

    def zero_grad(self):
        for p in self.parameters():
            p.zero_grad()

    def compile(self):
        """Mark for CUDA-graph capture (`Sequential` captures its forward on the first CUDA call)."""
        self._compiled = True
        return self

    # ---- hooks
    def register_forward_pre_hook(self, fn: Callable):
        self._fwd_pre_hooks.append(fn)
        return fn

    def register_forward_hook(self, fn: Callable):
        self._fwd_hooks.append(fn)
        return fn

    def __call__(self, *args, **kw):
        for h in self._fwd_pre_hooks:
            r = h(self, args[0] if args else None)
            if r is not None:
                args = (r,) + tuple(args[1:])
        out = self.forward(*args, **kw)
        for h in self._fwd_hooks:
            r = h(self, args[0] if args else None, out)
            if r is not None:
                out = r
        return out


def _param(t: torch.Tensor) -> Tensor:
    return Tensor(t.requires_grad_(True))


def _kaiming_uniform(out_f: int, in_f: int) -> torch.Tensor:
    # kaiming-uniform with a = sqrt(5) -> U(-1/sqrt(in), 1/sqrt(in)), as src/nn/nn_utils.h:13-42
    bound = 1.0 / math.sqrt(in_f) if in_f > 0 else 0.0
    return torch.empty(out_f, in_f).uniform_(-bound, bound)


class Linear(Module):
    """y = x W^T + b with W [out, in].  After `quantization.quantize_linear` the weight holds int8 codes with
    one scale per row and is dequantised on the fly (src/nn/linear.cpp:8-49)."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.weight = _param(_kaiming_uniform(out_features, in_features))
        bound = 1.0 / math.sqrt(in_features) if in_features > 0 else 0.0
        self.bias = _param(torch.empty(out_features).uniform_(-bound, bound)) if bias else None
        self.scales: Optional[Tensor] = None

    def forward(self, x: Tensor) -> Tensor:
        w = _unwrap(self.weight)
        xt = _unwrap(x)
        if self.scales is not None:
            w = w.to(xt.dtype) * _unwrap(self.scales).to(xt.dtype)[:, None]
        from ..amp import AutocastGuard
        b = _unwrap(self.bias) if self.bias is not None else None
        if AutocastGuard.is_enabled():
            dt = AutocastGuard.torch_dtype()
            xt, w = xt.to(dt), w.to(dt)
            b = b.to(dt) if b is not None else None
        return Tensor(Fn.linear(xt, w, b))


class QLoRALinear(Module):
    """Frozen NF4 base weight (absmax-scaled per row, dequantised every forward) + trainable LoRA A/B with
    scaling alpha/r (src/nn/qlora.cpp:10-69)."""

    def __init__(self, in_features: int, out_features: int, r: int = 8, lora_alpha: float = 16.0, has_bias: bool = True):
        super().__init__()
        from ..quantization import NF4_CODEBOOK, _nearest_code
        w = _kaiming_uniform(out_features, in_features)
        self.absmax = Tensor(w.abs().amax(1, keepdim=True).clamp_min(1e-8))
        self.base_codes = Tensor(_nearest_code(w / _unwrap(self.absmax), NF4_CODEBOOK), DataType.NF4)
        self.lora_A = _param(_kaiming_uniform(r, in_features))
        self.lora_B = _param(torch.zeros(out_features, r))
        self.bias = _param(torch.zeros(out_features)) if has_bias else None
        self.scaling = lora_alpha / r

    def base_weight(self) -> torch.Tensor:
        from ..quantization import NF4_CODEBOOK
        codes = _unwrap(self.base_codes)
        return NF4_CODEBOOK.to(codes.device)[codes.long()] * _unwrap(self.absmax)

    @property
    def weight(self) -> Tensor:
        """The frozen base weight: its NF4 codes (the reference binds the quantised tensor under this name)."""
        return self.base_codes

    def forward(self, x: Tensor) -> Tensor:
        xt = _unwrap(x)
        y = torch.nn.functional.linear(xt, self.base_weight().to(xt.dtype))
        y = y + torch.nn.functional.linear(torch.nn.functional.linear(xt, _unwrap(self.lora_A).to(xt.dtype)),
                                           _unwrap(self.lora_B).to(xt.dtype)) * self.scaling
        if self.bias is not None:
            y = y + _unwrap(self.bias).to(xt.dtype)
        return Tensor(y)


class Embedding(Module):
    """Rows of an N(0,1)-initialised table; indices may be floats (src/nn/embedding.cpp:30-160)."""

    def __init__(self, num_embeddings: int, embedding_dim: int):
        super().__init__()
        self.num_embeddings, self.embedding_dim = num_embeddings, embedding_dim
        self.weight = _param(torch.randn(num_embeddings, embedding_dim))

    def forward(self, idx: Tensor) -> Tensor:
        return Tensor(Fn.embedding(_unwrap(idx).to(torch.int64), _unwrap(self.weight)))


class LayerNorm(Module):
    def __init__(self, normalized_shape: Sequence[int], eps: float = 1e-5):
        super().__init__()
        self.normalized_shape, self.eps = ([int(normalized_shape)] if isinstance(normalized_shape, int) else list(normalized_shape)), eps
        self.weight = _param(torch.ones(*self.normalized_shape))
        self.bias = _param(torch.zeros(*self.normalized_shape))

    def forward(self, x: Tensor) -> Tensor:
        return Ops.layer_norm(x, self.normalized_shape, self.weight, self.bias, self.eps)


class RMSNorm(Module):
    def __init__(self, dim: int, eps: float = 1e-5):
        super().__init__()
        self.eps = eps
        self.weight = _param(torch.ones(dim))

    def forward(self, x: Tensor, residual: Optional[Tensor] = None) -> Tensor:
        return Ops.rms_norm(x, self.weight, self.eps, residual)


class BatchNorm2d(Module):
    def __init__(self, num_features: int, eps: float = 1e-5, momentum: float = 0.1):
        super().__init__()
        self.num_features, self.eps, self.momentum = num_features, eps, momentum
        self.weight = _param(torch.ones(num_features))
        self.bias = _param(torch.zeros(num_features))
        self.running_mean = Tensor(torch.zeros(num_features))
        self.running_var = Tensor(torch.ones(num_features))

    def forward(self, x: Tensor) -> Tensor:
        return Ops.batch_norm2d(x, self.running_mean, self.running_var, self.weight, self.bias, self.training, self.momentum, self.eps)


class Conv2d(Module):
    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, has_bias=True):
        super().__init__()
        self.stride, self.padding = stride, padding
        fan_in = in_channels * kernel_size * kernel_size
        bound = 1.0 / math.sqrt(fan_in)
        self.weight = _param(torch.empty(out_channels, in_channels, kernel_size, kernel_size).uniform_(-bound, bound))
        self.bias = _param(torch.empty(out_channels).uniform_(-bound, bound)) if has_bias else None

    def forward(self, x):
        return Ops.conv2d(x, self.weight, self.bias, self.stride, self.padding)


class Conv3d(Module):
    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, has_bias=True):
        super().__init__()
        self.stride, self.padding = stride, padding
        fan_in = in_channels * kernel_size ** 3
        bound = 1.0 / math.sqrt(fan_in)
        self.weight = _param(torch.empty(out_channels, in_channels, kernel_size, kernel_size, kernel_size).uniform_(-bound, bound))
        self.bias = _param(torch.empty(out_channels).uniform_(-bound, bound)) if has_bias else None

    def forward(self, x):
        return Ops.conv3d(x, self.weight, self.bias, self.stride, self.padding)


class MaxPool2d(Module):
    def __init__(self, kernel_size, stride=-1, padding=0):
        super().__init__()
        self.kernel_size, self.stride, self.padding = kernel_size, stride, padding

    def forward(self, x):
        return Ops.max_pool2d(x, self.kernel_size, self.stride, self.padding)


class MaxPool3d(Module):
    def __init__(self, kernel_size, stride=-1, padding=0):
        super().__init__()
        self.kernel_size, self.stride, self.padding = kernel_size, stride, padding

    def forward(self, x):
        return Ops.max_pool3d(x, self.kernel_size, self.stride, self.padding)


class AdaptiveAvgPool2d(Module):
    def __init__(self, output_height, output_width):
        super().__init__()
        self.output_height, self.output_width = output_height, output_width

    def forward(self, x):
        return Ops.adaptive_avg_pool2d(x, self.output_height, self.output_width)


class Dropout(Module):
    def __init__(self, p: float = 0.5):
        super().__init__()
        self.p = p

    def forward(self, x):
        return Tensor(Fn.dropout(_unwrap(x), self.p, self.training))


def _act(name, fn):
    class _A(Module):
        def forward(self, x):
            return fn(x)
    _A.__name__ = _A.__qualname__ = name
    return _A


ReLU = _act("ReLU", Ops.relu)
Sigmoid = _act("Sigmoid", Ops.sigmoid)
Tanh = _act("Tanh", Ops.tanh)
GELU = _act("GELU", Ops.gelu)
SiLU = _act("SiLU", Ops.silu)
SwiGLU = _act("SwiGLU", Ops.swiglu)


class LeakyReLU(Module):
    def __init__(self, negative_slope: float = 0.01):
        super().__init__()
        self.negative_slope = negative_slope

    def forward(self, x):
        return Ops.leaky_relu(x, self.negative_slope)


class Softmax(Module):
    def __init__(self, dim: int = -1):
        super().__init__()
        self.dim = dim

    def forward(self, x):
        return Ops.softmax(x, self.dim)


class Flatten(Module):
    def forward(self, x):
        t = _unwrap(x)
        return Tensor(t.reshape(t.shape[0], -1))


class Sequential(Module):
    """Container; after `compile()` the first CUDA forward is captured into a CUDA graph and later calls with the
    same input shape replay it (the reference replays and then runs eagerly again: src/nn/container.cpp:13-41)."""

    def __init__(self, modules: Optional[Sequence[Module]] = None):
        super().__init__()
        self.modules = list(modules) if modules else []
        self._graph = None

    def add(self, m: Module):
        self.modules.append(m)
        return self

    def _run(self, x):
        for m in self.modules:
            x = m(x)
        return x

    def forward(self, x):
        xt = _unwrap(x)
        if self._compiled and xt.is_cuda and not torch.is_grad_enabled():
            key = (tuple(xt.shape), xt.dtype)
            if self._graph is None or self._graph[0] != key:
                from ..cuda import CapturedGraph
                static_in = xt.clone()
                s = torch.cuda.Stream()
                s.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(s):
                    self._run(Tensor(static_in))  # warm-up outside capture (allocations, lazy inits)
                torch.cuda.current_stream().wait_stream(s)
                g = CapturedGraph()
                with g.capture():
                    static_out = _unwrap(self._run(Tensor(static_in)))
                self._graph = (key, g, static_in, static_out)
            _, g, static_in, static_out = self._graph
            static_in.copy_(xt)
            g.replay()
            return Tensor(static_out.clone())
        return self._run(x)


class MSELoss(Module):
    def forward(self, x, y): return Ops.mse_loss(x, y)


class CrossEntropyLoss(Module):
    def forward(self, x, y): return Ops.cross_entropy_loss(x, y)


class BCELoss(Module):
    def forward(self, x, y): return Ops.bce_loss(x, y)


class L1Loss(Module):
    def forward(self, x, y): return Ops.l1_loss(x, y)


class MultiHeadAttention(Module):
    """Four Linear layers around flash attention on [B, H, T, hd] (src/nn/attention.cpp:9-92)."""

    def __init__(self, embed_dim: int, num_heads: int, is_causal: bool = False):
        super().__init__()
        self.embed_dim, self.num_heads, self.head_dim, self.is_causal = embed_dim, num_heads, embed_dim // num_heads, is_causal
        self.q_proj, self.k_proj = Linear(embed_dim, embed_dim), Linear(embed_dim, embed_dim)
        self.v_proj, self.out_proj = Linear(embed_dim, embed_dim), Linear(embed_dim, embed_dim)

    def forward(self, query: Tensor, key: Optional[Tensor] = None, value: Optional[Tensor] = None) -> Tensor:
        key = key if key is not None else query
        value = value if value is not None else key
        B, Tq, _ = query.shape
        Tk = key.shape[1]
        q = _unwrap(self.q_proj(query)).view(B, Tq, self.num_heads, self.head_dim)
        k = _unwrap(self.k_proj(key)).view(B, Tk, self.num_heads, self.head_dim)
        v = _unwrap(self.v_proj(value)).view(B, Tk, self.num_heads, self.head_dim)
        o = Fn.flash_attention_bthd(q, k, v, causal=self.is_causal)
        return self.out_proj(Tensor(o.reshape(B, Tq, self.embed_dim)))


class TransformerDecoderLayer(Module):
    """Post-LN decoder block: self-attention -> add & LayerNorm -> optional cross-attention -> GELU FFN -> add &
    LayerNorm, the two add+norm steps fused (src/nn/transformer.cpp:7-70)."""

    def __init__(self, embed_dim: int, num_heads: int, dim_feedforward: int = 2048):
        super().__init__()
        self.self_attn = MultiHeadAttention(embed_dim, num_heads)
        self.cross_attn = MultiHeadAttention(embed_dim, num_heads)
        self.norm1, self.norm2, self.norm3 = LayerNorm([embed_dim]), LayerNorm([embed_dim]), LayerNorm([embed_dim])
        self.linear1, self.linear2 = Linear(embed_dim, dim_feedforward), Linear(dim_feedforward, embed_dim)

    @property
    def multihead_attn(self):
        """The cross-attention block under the reference's member name (include/litetorch/nn.h)."""
        return self.cross_attn

    def forward(self, x: Tensor, memory: Optional[Tensor] = None) -> Tensor:
        a = self.self_attn(x)
        x = Ops.fused_add_layernorm(a, x, self.norm1.normalized_shape, self.norm1.weight, self.norm1.bias, self.norm1.eps)
        if memory is not None:
            c = self.cross_attn(x, memory, memory)
            x = Ops.fused_add_layernorm(c, x, self.norm2.normalized_shape, self.norm2.weight, self.norm2.bias, self.norm2.eps)
        h = _unwrap(self.linear1.weight)
        f = Tensor(Fn.linear(_unwrap(x), h, _unwrap(self.linear1.bias), act="gelu"))
        f = self.linear2(f)
        return Ops.fused_add_layernorm(f, x, self.norm3.normalized_shape, self.norm3.weight, self.norm3.bias, self.norm3.eps)


class LlamaMLP(Module):
    """SwiGLU feed-forward: down(silu(gate(x)) * up(x)) with gate and up fused into one [2F, d] projection."""

    def __init__(self, dim: int, ffn: int):
        super().__init__()
        self.gate_up = Linear(dim, 2 * ffn, bias=False)
        self.down = Linear(ffn, dim, bias=False)

    def forward(self, x):
        return self.down(Ops.swiglu(self.gate_up(x)))


class GQAttention(Module):
    """Causal grouped-query attention with interleaved RoPE on a fused QKV projection."""

    def __init__(self, dim: int, n_heads: int, n_kv_heads: int, head_dim: Optional[int] = None, rope_theta: float = 1e4,
                 max_seq: int = 4096):
        super().__init__()
        self.n_heads, self.n_kv, self.hd = n_heads, n_kv_heads, head_dim or dim // n_heads
        self.wqkv = Linear(dim, (n_heads + 2 * n_kv_heads) * self.hd, bias=False)
        self.wo = Linear(n_heads * self.hd, dim, bias=False)
        inv = 1.0 / (rope_theta ** (torch.arange(0, self.hd, 2, dtype=torch.float64) / self.hd))
        ang = torch.arange(max_seq, dtype=torch.float64)[:, None] * inv[None]
        self.cos, self.sin = Tensor(ang.cos().float()), Tensor(ang.sin().float())

    def forward(self, x):
        B, T, _ = x.shape
        qkv = _unwrap(self.wqkv(x))
        H, Hk, hd = self.n_heads, self.n_kv, self.hd
        q = qkv[..., :H * hd].view(B, T, H, hd).transpose(1, 2)
        k = qkv[..., H * hd:(H + Hk) * hd].view(B, T, Hk, hd).transpose(1, 2)
        v = qkv[..., (H + Hk) * hd:].view(B, T, Hk, hd).transpose(1, 2)
        cos, sin = _unwrap(self.cos)[:T].to(qkv.device), _unwrap(self.sin)[:T].to(qkv.device)
        q, k = Fn.rope(q, cos, sin), Fn.rope(k, cos, sin)
        o = Fn.flash_attention(q, k, v, is_causal=True)
        return self.wo(Tensor(o.transpose(1, 2).reshape(B, T, H * hd)))


from .moe import MoELinear  # noqa: E402
from ..parallel.tp import ColumnParallelLinear, RowParallelLinear  # noqa: E402
from ..serving import (GuidedDecoder, MedusaEngine, MedusaHead, PrefixCache, Request, ServingScheduler,  # noqa: E402
                       SpeculativeEngine)

__all__ = [n for n in dir() if not n.startswith("_")]
