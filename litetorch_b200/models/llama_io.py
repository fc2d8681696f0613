"""Weights of Hugging Face Llama checkpoints in and out of the Llama engine.

The engine keeps three things differently from the `transformers` layout, all of them pure re-arrangements:

* q, k and v projections are one matrix `wqkv` with rows [all q heads | all kv heads of k | all kv heads of v];
  gate and up projections are one matrix `w_gu` with rows [gate | up];
* rotary embedding pairs are interleaved (dimensions 2i and 2i + 1 rotate together) where `transformers` pairs
  dimension i with i + head_dim / 2, so the rows of every q and k head are permuted (scores are dot products over the
  head dimension and do not change when q and k are permuted alike);
* names (`embed`, `layers.N.attn_norm`, ..., `final_norm`, `lm_head`).

`from_hf` / `to_hf` convert a state dict, `config_from_hf` / `config_to_hf` the hyper-parameters, `load_pretrained` /
`save_pretrained` read and write a directory of `*.safetensors` files with its `config.json`.  The reference has no
counterpart (it cannot load third-party checkpoints); the conversions are checked against `transformers`' own Llama
forward pass in tests/test_llama_io_cpu.py.
"""
from __future__ import annotations

import json
import os
from typing import Dict, List

import torch

from .llama import LlamaConfig, param_specs


def config_from_hf(hf) -> LlamaConfig:
    """`hf`: a `transformers.LlamaConfig` or the dict of a `config.json`."""
    g = (lambda k, d=None: hf.get(k, d)) if isinstance(hf, dict) else (lambda k, d=None: getattr(hf, k, d))
    heads = int(g("num_attention_heads"))
    hidden = int(g("hidden_size"))
    if g("attention_bias", False) or g("mlp_bias", False):
        raise ValueError("the engine's linear layers have no bias")
    scaling = g("rope_scaling")
    if scaling and (scaling.get("rope_type") or scaling.get("type")) not in (None, "default"):
        raise ValueError("rope scaling %r is not supported (plain rotary embedding only)" % (scaling,))
    theta = g("rope_theta")
    if theta is None:                                   # newer configs keep it under rope_parameters
        theta = (g("rope_parameters") or {}).get("rope_theta", 1e4)
    return LlamaConfig(vocab_size=int(g("vocab_size")), n_layers=int(g("num_hidden_layers")), d_model=hidden, n_heads=heads,
                       n_kv_heads=int(g("num_key_value_heads") or heads), head_dim=int(g("head_dim") or hidden // heads),
                       ffn=int(g("intermediate_size")), rms_eps=float(g("rms_norm_eps", 1e-5)), rope_theta=float(theta),
                       max_seq=int(g("max_position_embeddings", 2048)), name=str(g("_name_or_path", "") or "llama-hf"))


def config_to_hf(cfg: LlamaConfig) -> dict:
    return {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "vocab_size": cfg.vocab_size,
            "hidden_size": cfg.d_model, "intermediate_size": cfg.ffn, "num_hidden_layers": cfg.n_layers,
            "num_attention_heads": cfg.n_heads, "num_key_value_heads": cfg.n_kv_heads, "head_dim": cfg.head_dim,
            "rms_norm_eps": cfg.rms_eps, "rope_theta": cfg.rope_theta, "max_position_embeddings": cfg.max_seq,
            "hidden_act": "silu", "tie_word_embeddings": False, "attention_bias": False, "mlp_bias": False,
            "torch_dtype": "float32"}


def _to_interleaved(w: torch.Tensor, heads: int, hd: int) -> torch.Tensor:
    """Rows of every head from [first halves | second halves] to interleaved pairs."""
    cols = w.shape[1]
    return w.view(heads, 2, hd // 2, cols).transpose(1, 2).reshape(heads * hd, cols)


def _to_half_split(w: torch.Tensor, heads: int, hd: int) -> torch.Tensor:
    cols = w.shape[1]
    return w.view(heads, hd // 2, 2, cols).transpose(1, 2).reshape(heads * hd, cols)


def from_hf(cfg: LlamaConfig, state: Dict[str, torch.Tensor]) -> List[torch.Tensor]:
    """The engine's parameters, in `param_specs(cfg)` order, from a `LlamaForCausalLM` state dict."""
    def get(name):
        for k in (name, "model." + name):
            if k in state:
                return state[k].detach().to(torch.float32)
        raise KeyError("the checkpoint has no tensor %r" % name)

    embed = get("model.embed_tokens.weight") if "model.embed_tokens.weight" in state else get("embed_tokens.weight")
    out = {"embed": embed, "final_norm": get("model.norm.weight") if "model.norm.weight" in state else get("norm.weight"),
           "lm_head": state["lm_head.weight"].detach().float() if "lm_head.weight" in state else embed}   # tied embeddings
    hd = cfg.head_dim
    for i in range(cfg.n_layers):
        h, p = "model.layers.%d." % i, "layers.%d." % i
        q = _to_interleaved(get(h + "self_attn.q_proj.weight"), cfg.n_heads, hd)
        k = _to_interleaved(get(h + "self_attn.k_proj.weight"), cfg.n_kv_heads, hd)
        out[p + "wqkv"] = torch.cat([q, k, get(h + "self_attn.v_proj.weight")], 0)
        out[p + "wo"] = get(h + "self_attn.o_proj.weight")
        out[p + "w_gu"] = torch.cat([get(h + "mlp.gate_proj.weight"), get(h + "mlp.up_proj.weight")], 0)
        out[p + "w_down"] = get(h + "mlp.down_proj.weight")
        out[p + "attn_norm"] = get(h + "input_layernorm.weight")
        out[p + "mlp_norm"] = get(h + "post_attention_layernorm.weight")
    tensors = []
    for s in param_specs(cfg):
        t = out[s.name]
        if tuple(t.shape) != tuple(s.shape):
            raise ValueError("%s: the checkpoint gives %s, the configuration expects %s" % (s.name, tuple(t.shape), tuple(s.shape)))
        tensors.append(t.contiguous())
    return tensors


def to_hf(cfg: LlamaConfig, tensors: List[torch.Tensor]) -> Dict[str, torch.Tensor]:
    """A `LlamaForCausalLM` state dict from the engine's parameters (`engine.w.parameters()`)."""
    by = {s.name: t.detach().to(torch.float32).view(*s.shape) for s, t in zip(param_specs(cfg), tensors)}
    hd, nq, nkv = cfg.head_dim, cfg.n_heads * cfg.head_dim, cfg.n_kv_heads * cfg.head_dim
    sd = {"model.embed_tokens.weight": by["embed"], "model.norm.weight": by["final_norm"], "lm_head.weight": by["lm_head"]}
    for i in range(cfg.n_layers):
        h, p = "model.layers.%d." % i, "layers.%d." % i
        wqkv, wgu = by[p + "wqkv"], by[p + "w_gu"]
        sd[h + "self_attn.q_proj.weight"] = _to_half_split(wqkv[:nq], cfg.n_heads, hd)
        sd[h + "self_attn.k_proj.weight"] = _to_half_split(wqkv[nq:nq + nkv], cfg.n_kv_heads, hd)
        sd[h + "self_attn.v_proj.weight"] = wqkv[nq + nkv:]
        sd[h + "self_attn.o_proj.weight"] = by[p + "wo"]
        sd[h + "mlp.gate_proj.weight"] = wgu[:cfg.ffn]
        sd[h + "mlp.up_proj.weight"] = wgu[cfg.ffn:]
        sd[h + "mlp.down_proj.weight"] = by[p + "w_down"]
        sd[h + "input_layernorm.weight"] = by[p + "attn_norm"]
        sd[h + "post_attention_layernorm.weight"] = by[p + "mlp_norm"]
    return {k: v.contiguous().clone() for k, v in sd.items()}


def load_into(engine, state: Dict[str, torch.Tensor]) -> None:
    """Put a Hugging Face state dict into an engine's weight provider (whole on one device, or sharded: every rank is
    given the same state dict and keeps its part).  The optimizer's moments are left as they are."""
    engine.w.load_parameters(from_hf(engine.cfg, state))


def read_state_dict(directory: str) -> Dict[str, torch.Tensor]:
    """Every tensor of the `*.safetensors` files in `directory` (the index file, if any, is not needed)."""
    from safetensors.torch import load_file
    files = sorted(f for f in os.listdir(directory) if f.endswith(".safetensors"))
    if not files:
        raise FileNotFoundError("no .safetensors file in %s" % directory)
    state: Dict[str, torch.Tensor] = {}
    for f in files:
        state.update(load_file(os.path.join(directory, f)))
    return state


def load_pretrained(directory: str, device="cuda", **engine_kw):
    """An engine with unsharded weights from a Hugging Face model directory (`config.json` + `*.safetensors`)."""
    from .llama import LlamaEngine
    with open(os.path.join(directory, "config.json")) as f:
        cfg = config_from_hf(json.load(f))
    engine = LlamaEngine(cfg, device, **engine_kw)
    load_into(engine, read_state_dict(directory))
    return engine


def save_pretrained(engine, directory: str, dtype=torch.bfloat16) -> None:
    """Write the engine's weights as `model.safetensors` + `config.json` that `transformers` loads.  With sharded
    weights every rank calls this (the gather is a collective) and rank 0 writes."""
    from safetensors.torch import save_file
    tensors = engine.w.parameters()
    rank = int(os.environ.get("RANK", "0")) if getattr(engine.w, "world", 1) > 1 else 0
    if rank != 0:
        return
    os.makedirs(directory, exist_ok=True)
    sd = {k: v.to("cpu", dtype).contiguous() for k, v in to_hf(engine.cfg, [t.cpu() for t in tensors]).items()}
    save_file(sd, os.path.join(directory, "model.safetensors.tmp"), metadata={"format": "pt"})
    os.replace(os.path.join(directory, "model.safetensors.tmp"), os.path.join(directory, "model.safetensors"))
    cfg = config_to_hf(engine.cfg)
    cfg["torch_dtype"] = str(dtype).replace("torch.", "")
    with open(os.path.join(directory, "config.json.tmp"), "w") as f:
        json.dump(cfg, f, indent=1)
    os.replace(os.path.join(directory, "config.json.tmp"), os.path.join(directory, "config.json"))
