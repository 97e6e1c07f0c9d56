"""Export of a merged GPT checkpoint to the state dict of `transformers.GPT2LMHeadModel`.

The GPT of this framework and GPT-2 are the same network (learned positions, pre-LayerNorm blocks, fused QKV
projection split into [Q | K | V] thirds with the heads inside each third, tanh-approximated GeLU, final LayerNorm,
LM head tied to the word embeddings), so the export is a renaming plus a transpose of every linear layer (GPT-2
stores them as [in, out]).  Besides interoperability this gives an independent implementation to compare logits
against (tests/test_checkpoint_cpu.py).
"""
from __future__ import annotations

from typing import Dict, Sequence

import torch


def to_hf_gpt2(full: Dict[str, torch.Tensor], op_names: Sequence[str]) -> Dict[str, torch.Tensor]:
    """`full`: unsharded fp32 tensors keyed '{global op index}.{param}' (runtime/checkpointing.merge_tp_shards)."""
    sd: Dict[str, torch.Tensor] = {}
    layer = -1
    for i, op in enumerate(op_names):
        def get(p):
            return full[f"{i}.{p}"].float()
        if op == "encoder-embedding":
            sd["transformer.wte.weight"] = get("word_embeddings.weight")
            sd["transformer.wpe.weight"] = get("position_embeddings.weight")
            sd["lm_head.weight"] = sd["transformer.wte.weight"]
        elif op == "enc-1st-layernorm":
            layer += 1
            sd[f"transformer.h.{layer}.ln_1.weight"], sd[f"transformer.h.{layer}.ln_1.bias"] = \
                get("layernorm.weight"), get("layernorm.bias")
        elif op == "enc-attention-qkv":
            w = get("query_key_value.weight")
            sd[f"transformer.h.{layer}.attn.c_attn.weight"] = w.reshape(-1, w.shape[-1]).t().contiguous()
            sd[f"transformer.h.{layer}.attn.c_attn.bias"] = get("query_key_value.bias").reshape(-1)
        elif op == "enc-attention-dense":
            sd[f"transformer.h.{layer}.attn.c_proj.weight"] = get("dense.weight").t().contiguous()
            sd[f"transformer.h.{layer}.attn.c_proj.bias"] = get("dense.bias")
        elif op == "enc-2nd-layernorm":
            sd[f"transformer.h.{layer}.ln_2.weight"], sd[f"transformer.h.{layer}.ln_2.bias"] = \
                get("layernorm.weight"), get("layernorm.bias")
        elif op == "enc-MLP-GEMM-1":
            sd[f"transformer.h.{layer}.mlp.c_fc.weight"] = get("dense_h_to_4h.weight").t().contiguous()
            sd[f"transformer.h.{layer}.mlp.c_fc.bias"] = get("dense_h_to_4h.bias")
        elif op == "enc-MLP-GEMM-2":
            sd[f"transformer.h.{layer}.mlp.c_proj.weight"] = get("dense_4h_to_h.weight").t().contiguous()
            sd[f"transformer.h.{layer}.mlp.c_proj.bias"] = get("dense_4h_to_h.bias")
        elif op == "final-layernorm":
            sd["transformer.ln_f.weight"], sd["transformer.ln_f.bias"] = get("layernorm.weight"), get("layernorm.bias")
    return sd


def hf_gpt2_config(cfg):
    """`transformers.GPT2Config` of a GPTConfig of this framework (dropout off: the export is for inference)."""
    from transformers import GPT2Config
    assert cfg.heads * cfg.head_dim == cfg.hidden, "GPT-2 ties the head size to hidden / heads"
    return GPT2Config(vocab_size=cfg.padded_vocab, n_positions=cfg.max_positions, n_embd=cfg.hidden,
                      n_layer=cfg.num_layers, n_head=cfg.heads, n_inner=cfg.ffn, activation_function="gelu_new",
                      layer_norm_epsilon=cfg.layernorm_eps, resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0)
