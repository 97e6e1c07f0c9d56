"""Conversion between this framework's op-indexed parameter names and the parameter names of an upstream
Megatron-LM GPT checkpoint (a single, unsharded state dict).

The reference stores parameters under ``language_model.ops.{i}.…`` (runtime/megatron/model/flex_model.py:378),
which no upstream tool reads.  `merge_tp_shards` (runtime/checkpointing.py) rebuilds full tensors keyed
``{global op index}.{param}``; the functions here rename those to

    language_model.embedding.{word,position}_embeddings.weight
    language_model.encoder.layers.{l}.{input_layernorm | self_attention.query_key_value | self_attention.dense |
                                       post_attention_layernorm | mlp.dense_h_to_4h | mlp.dense_4h_to_h}.{weight,bias}
    language_model.encoder.final_layernorm.{weight,bias}

(`legacy=True`: ``transformer`` / ``attention`` instead of ``encoder`` / ``self_attention``, the names used before
Megatron-LM 2.5) and back.  The fused QKV projection is stored here as [Q heads | K heads | V heads]; upstream
checkpoint version 3.0 interleaves per head ([head][q, k, v][head_dim]), so the rows are permuted on the way.
"""
from __future__ import annotations

from typing import Dict, List, Sequence

import torch

_LAYER_PARAMS = {
    "enc-1st-layernorm": ("input_layernorm", ("layernorm.weight", "layernorm.bias")),
    "enc-attention-qkv": ("{attn}.query_key_value", ("query_key_value.weight", "query_key_value.bias")),
    "enc-attention-dense": ("{attn}.dense", ("dense.weight", "dense.bias")),
    "enc-2nd-layernorm": ("post_attention_layernorm", ("layernorm.weight", "layernorm.bias")),
    "enc-MLP-GEMM-1": ("mlp.dense_h_to_4h", ("dense_h_to_4h.weight", "dense_h_to_4h.bias")),
    "enc-MLP-GEMM-2": ("mlp.dense_4h_to_h", ("dense_4h_to_h.weight", "dense_4h_to_h.bias")),
}


def _name_map(op_names: Sequence[str], legacy: bool) -> Dict[str, str]:
    """ours ('{op index}.{param}') -> upstream name."""
    enc, attn = ("transformer", "attention") if legacy else ("encoder", "self_attention")
    out: Dict[str, str] = {}
    layer = -1
    for i, op in enumerate(op_names):
        if op == "encoder-embedding":
            out[f"{i}.word_embeddings.weight"] = "language_model.embedding.word_embeddings.weight"
            out[f"{i}.position_embeddings.weight"] = "language_model.embedding.position_embeddings.weight"
        elif op == "final-layernorm":
            for p in ("weight", "bias"):
                out[f"{i}.layernorm.{p}"] = f"language_model.{enc}.final_layernorm.{p}"
        elif op in _LAYER_PARAMS:
            if op == "enc-1st-layernorm":
                layer += 1
            module, params = _LAYER_PARAMS[op]
            for p in params:
                out[f"{i}.{p}"] = f"language_model.{enc}.layers.{layer}.{module.format(attn=attn)}.{p.rsplit('.', 1)[1]}"
    return out


def _qkv_to_upstream(t: torch.Tensor, heads: int) -> torch.Tensor:
    """[3, heads * hd, ...] (Q | K | V blocks) -> [heads * 3 * hd, ...] (q, k, v per head)."""
    rest = tuple(t.shape[2:])
    hd = t.shape[1] // heads
    return t.reshape(3, heads, hd, *rest).transpose(0, 1).reshape(heads * 3 * hd, *rest).contiguous()


def _qkv_from_upstream(t: torch.Tensor, heads: int) -> torch.Tensor:
    rest = tuple(t.shape[1:])
    hd = t.shape[0] // (3 * heads)
    return t.reshape(heads, 3, hd, *rest).transpose(0, 1).reshape(3, heads * hd, *rest).contiguous()


def export_megatron_gpt(full: Dict[str, torch.Tensor], op_names: Sequence[str], heads: int,
                        legacy: bool = False) -> Dict[str, torch.Tensor]:
    """`full`: unsharded tensors keyed '{global op index}.{param}' -> upstream-named state dict."""
    names = _name_map(op_names, legacy)
    out = {}
    for ours, theirs in names.items():
        if ours not in full:
            continue          # the tied LM-head copy of the word embeddings has no entry of its own upstream
        t = full[ours]
        out[theirs] = _qkv_to_upstream(t, heads) if "query_key_value" in ours else t
    missing = [k for k in full if k not in names and "word_embeddings" not in k]
    if missing:
        raise KeyError(f"no upstream name for {missing[:4]}")
    return out


def import_megatron_gpt(sd: Dict[str, torch.Tensor], op_names: Sequence[str], heads: int,
                        legacy: bool = False) -> Dict[str, torch.Tensor]:
    """Inverse of export_megatron_gpt: upstream-named state dict -> tensors keyed '{global op index}.{param}'."""
    out = {}
    for ours, theirs in _name_map(op_names, legacy).items():
        t = sd[theirs]
        out[ours] = _qkv_from_upstream(t, heads) if "query_key_value" in ours else t
    return out


def upstream_names(op_names: Sequence[str], legacy: bool = False) -> List[str]:
    return list(_name_map(op_names, legacy).values())
