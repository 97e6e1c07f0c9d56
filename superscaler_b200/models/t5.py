"""T5 (encoder-decoder) as a flat op list with the reference's op names
(runtime/megatron/model/flex_t5.py:20-72): `encoder-embedding`, 13 ops per encoder layer,
`enc-final-layernorm`, `decoder-embedding`, 21 ops per decoder layer (causal self-attention, cross-attention
over the encoder output, MLP), `dec-final-layernorm`, `t5-post-process`  -- 821 ops for 24 + 24 layers.

Like the reference's T5 the model uses learned absolute position embeddings shared by encoder and
decoder, and ties the LM head to the word embeddings.  The MLP activation is configurable
(tanh-GeLU as in the reference, or ReLU).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List


from ..ops import functional as F
from .base import Env, Op, OpInfo
from .gpt import GPT_LAYER_OPS
from .transformer_ops import (AttnDropoutOp, BiasActOp, BiasDropoutAddOp, ContextOp, DenseOp, EmbeddingOp,
                              LayerNormOp, LMHeadLossOp, MLPUpOp, QKVOp, ScoreOp, SoftmaxOp)

T5_DEC_LAYER_OPS = ["dec-1st-layernorm", "dec-attention-qkv-1", "dec-attention-score-1", "dec-attention-softmax-1",
                    "dec-attention-dropout-1", "dec-attention-context-1", "dec-attention-dense-1",
                    "dec-post-attention-dropout-1", "dec-2nd-layernorm", "dec-attention-qkv-2",
                    "dec-attention-score-2", "dec-attention-softmax-2", "dec-attention-dropout-2",
                    "dec-attention-context-2", "dec-attention-dense-2", "dec-post-attention-dropout-2",
                    "dec-3rd-layernorm", "dec-MLP-GEMM-1", "dec-MLP-gelu", "dec-MLP-GEMM-2", "dec-post-MLP-dropout"]


@dataclass
class T5Config:
    num_layers: int = 24
    hidden: int = 1024
    heads: int = 16
    head_dim: int = 64
    ffn: int = 4096
    seq_length: int = 512          # encoder sequence
    dec_seq_length: int = 128
    vocab: int = 32128
    max_positions: int = 512
    hidden_dropout: float = 0.1
    attention_dropout: float = 0.1
    layernorm_eps: float = 1e-5
    init_std: float = 0.02
    activation: int = F.ACT_GELU
    make_vocab_divisible_by: int = 128
    max_tp: int = 8
    # T5 relative-position buckets in the self-attentions: one learned [heads, buckets] table per stack, added to the
    # scores through a per-head table over the distance key - query (the flash-attention kernels take that table);
    # off = learned absolute positions alone, as in the reference's T5.  A plan turns it on with
    # "relative_position_bias": true (the B200 definition of T5 770M does).
    relative_position_bias: bool = False
    relative_attention_num_buckets: int = 32
    relative_attention_max_distance: int = 128

    @property
    def padded_vocab(self) -> int:
        m = self.make_vocab_divisible_by * self.max_tp
        return (self.vocab + m - 1) // m * m

    @property
    def output_init_std(self) -> float:
        return self.init_std / (2.0 * self.num_layers) ** 0.5


def t5_op_names(num_layers: int) -> List[str]:
    return (["encoder-embedding"] + GPT_LAYER_OPS * num_layers + ["enc-final-layernorm", "decoder-embedding"] +
            T5_DEC_LAYER_OPS * num_layers + ["dec-final-layernorm", "t5-post-process"])


def t5_layer_of(index: int, num_layers: int) -> int:
    enc_end = 1 + 13 * num_layers
    if 1 <= index < enc_end:
        return (index - 1) // 13
    dec_start = enc_end + 2
    if dec_start <= index < dec_start + 21 * num_layers:
        return num_layers + (index - dec_start) // 21
    return -1


class DecoderEmbeddingOp(EmbeddingOp):
    """Embeds the decoder tokens; the encoder output that arrives as "x" continues as "enc_out"."""

    def __init__(self, info, env):
        super().__init__(info, env, ids_key="dec_ids", seq_attr="dec_seq_length")
        self.reads = ("dec_ids", "x")
        self.writes = ("x", "enc_out")

    def forward(self, st):
        enc = st["x"]
        super().forward(st)
        st["enc_out"] = enc


def build_t5_op(info: OpInfo, env: Env) -> Op:
    c = env.cfg
    n = info.name
    dec = n.startswith("dec-")
    seq = "dec_seq_length" if dec else "seq_length"
    proj = c.heads * c.head_dim
    if n == "encoder-embedding":
        return EmbeddingOp(info, env)
    if n == "decoder-embedding":
        return DecoderEmbeddingOp(info, env)
    if n.endswith("final-layernorm"):
        return LayerNormOp(info, env, keep_residual=False)
    if n.endswith("layernorm"):
        return LayerNormOp(info, env)
    if n in ("enc-attention-qkv", "dec-attention-qkv-1"):
        return QKVOp(info, env)
    if n == "dec-attention-qkv-2":
        return QKVOp(info, env, kind="cross")
    if n == "enc-attention-score":
        return ScoreOp(info, env, mode="full", sq_attr=seq, sk_attr=seq)
    if n == "dec-attention-score-1":
        return ScoreOp(info, env, mode="causal", sq_attr=seq, sk_attr=seq)
    if n == "dec-attention-score-2":
        return ScoreOp(info, env, mode="cross", sq_attr="dec_seq_length", sk_attr="seq_length")
    if "attention-softmax" in n:
        return SoftmaxOp(info, env, mode="causal" if n == "dec-attention-softmax-1" else "full")
    if "attention-dropout" in n and not n.startswith(("enc-post", "dec-post")):
        return AttnDropoutOp(info, env)
    if "attention-context" in n:
        return ContextOp(info, env)
    if "attention-dense" in n:
        return DenseOp(info, env, key="dense", in_features=proj, out_features=c.hidden)
    if "post-attention-dropout" in n or n.endswith("post-MLP-dropout"):
        return BiasDropoutAddOp(info, env)
    if n.endswith("MLP-GEMM-1"):
        return MLPUpOp(info, env)
    if n.endswith("MLP-gelu"):
        return BiasActOp(info, env)
    if n.endswith("MLP-GEMM-2"):
        return DenseOp(info, env, key="dense_4h_to_h", in_features=c.ffn, out_features=c.hidden)
    if n == "t5-post-process":
        return LMHeadLossOp(info, env)
    raise KeyError(f"unknown T5 op {n}")


def t5_config_from_plan(d: dict, **overrides) -> T5Config:
    cfg = T5Config(num_layers=d["num_layers"], hidden=d["hidden_size"], heads=d["num_attention_heads"],
                   head_dim=d["kv_channels"], ffn=d["ffn_hidden_size"], seq_length=d["encoder_seq_length"],
                   dec_seq_length=d["decoder_seq_length"], max_positions=d["max_position_embeddings"],
                   vocab=d.get("vocab_size", 30592))
    # optional keys of the B200 model definition (absent in plans of the reference's T5)
    if d.get("relative_position_bias"):
        cfg.relative_position_bias = True
        cfg.relative_attention_num_buckets = int(d.get("relative_attention_num_buckets", 32))
    if d.get("activation") in ("relu", "gelu"):
        cfg.activation = F.ACT_RELU if d["activation"] == "relu" else F.ACT_GELU
    for k, v in overrides.items():
        setattr(cfg, k, v)
    return cfg
