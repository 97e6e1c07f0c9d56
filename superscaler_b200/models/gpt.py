"""GPT as a flat op list: `encoder-embedding`, 13 ops per layer, `final-layernorm`, `gpt-post-process`
(315 ops for 24 layers), with the op names of the reference (runtime/megatron/model/flex_gpt.py:18-41) so
plans and the profiled database address the same ops.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List

from ..ops import functional as F
from .base import Env, Op, OpInfo
from .transformer_ops import (AttnDropoutOp, BiasActOp, BiasDropoutAddOp, ContextOp, DenseOp, EmbeddingOp,
                              LayerNormOp, LMHeadLossOp, MLPUpOp, QKVOp, ScoreOp, SoftmaxOp)

GPT_LAYER_OPS = ["enc-1st-layernorm", "enc-attention-qkv", "enc-attention-score", "enc-attention-softmax",
                 "enc-attention-dropout", "enc-attention-context", "enc-attention-dense",
                 "enc-post-attention-dropout", "enc-2nd-layernorm", "enc-MLP-GEMM-1", "enc-MLP-gelu",
                 "enc-MLP-GEMM-2", "enc-post-MLP-dropout"]


@dataclass
class GPTConfig:
    num_layers: int = 24
    hidden: int = 2048
    heads: int = 16
    head_dim: int = 128
    ffn: int = 8192
    seq_length: int = 2048
    vocab: int = 51200
    max_positions: int = 2048
    hidden_dropout: float = 0.1
    attention_dropout: float = 0.1
    layernorm_eps: float = 1e-5
    init_std: float = 0.02
    activation: int = F.ACT_GELU
    make_vocab_divisible_by: int = 128
    max_tp: int = 8

    @property
    def padded_vocab(self) -> int:
        # vocabulary padded to a multiple of 128 x the largest TP degree
        # (reference: runtime/megatron/tokenizer/tokenizer.py:54-71)
        m = self.make_vocab_divisible_by * self.max_tp
        return (self.vocab + m - 1) // m * m

    @property
    def output_init_std(self) -> float:
        return self.init_std / (2.0 * self.num_layers) ** 0.5


def gpt_op_names(num_layers: int) -> List[str]:
    return ["encoder-embedding"] + GPT_LAYER_OPS * num_layers + ["final-layernorm", "gpt-post-process"]


def gpt_layer_of(index: int, num_layers: int) -> int:
    if index == 0 or index > 13 * num_layers:
        return -1
    return (index - 1) // 13


def build_gpt_op(info: OpInfo, env: Env) -> Op:
    c = env.cfg
    n = info.name
    if n == "encoder-embedding":
        return EmbeddingOp(info, env)
    if n in ("enc-1st-layernorm", "enc-2nd-layernorm"):
        return LayerNormOp(info, env)
    if n == "final-layernorm":
        return LayerNormOp(info, env, keep_residual=False)
    if n == "enc-attention-qkv":
        return QKVOp(info, env)
    if n == "enc-attention-score":
        return ScoreOp(info, env, mode="causal")
    if n == "enc-attention-softmax":
        return SoftmaxOp(info, env, mode="causal")
    if n == "enc-attention-dropout":
        return AttnDropoutOp(info, env)
    if n == "enc-attention-context":
        return ContextOp(info, env)
    if n == "enc-attention-dense":
        return DenseOp(info, env, key="dense", in_features=c.heads * c.head_dim, out_features=c.hidden)
    if n in ("enc-post-attention-dropout", "enc-post-MLP-dropout"):
        return BiasDropoutAddOp(info, env)
    if n == "enc-MLP-GEMM-1":
        return MLPUpOp(info, env)
    if n == "enc-MLP-gelu":
        return BiasActOp(info, env)
    if n == "enc-MLP-GEMM-2":
        return DenseOp(info, env, key="dense_4h_to_h", in_features=c.ffn, out_features=c.hidden)
    if n == "gpt-post-process":
        return LMHeadLossOp(info, env)
    raise KeyError(f"unknown GPT op {n}")


def gpt_config_from_plan(d: dict, **overrides) -> GPTConfig:
    heads = d["num_attention_heads"]
    cfg = GPTConfig(num_layers=d["num_layers"], hidden=d["hidden_size"], heads=heads,
                    head_dim=d.get("kv_channels", d["hidden_size"] // heads), ffn=d.get("ffn_hidden_size", 4 * d["hidden_size"]),
                    seq_length=d["seq_length"], max_positions=d["max_position_embeddings"],
                    vocab=d.get("vocab_size", 51200))
    for k, v in overrides.items():
        setattr(cfg, k, v)
    return cfg
