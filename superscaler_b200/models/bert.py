"""BERT as a flat op list: `encoder-embedding` (word + position + token-type), 13 ops per layer (the same names as
the GPT / T5 encoder layers, so plans and profiled tables address them alike), `final-layernorm`, `bert-post-process`.

The reference's tree holds BERT's data side, inherited from Megatron-LM (runtime/megatron/data/bert_dataset.py,
dataset_utils.py, the WordPiece tokenizer, --bert-no-binary-head at runtime/megatron/arguments.py:319) but not the
model file it was written for.  The model here follows Megatron-LM's BERT (LM head = dense + GeLU + LayerNorm + tied
vocabulary projection; loss = masked-LM loss + sentence-order loss) as an op-list model like the others, so every
plan feature (per-op tensor / data parallel degrees, pipeline stages, recompute) applies.

  * attention looks both ways; padding is masked by the number of real tokens per sample (`enc_lens`);
  * the head transforms the hidden states (dense + GeLU + LayerNorm), projects them with the tied word embedding
    and averages the cross entropy over the masked positions (`loss_mask`);
  * with `binary_head` the first token of every sample goes through a tanh pooler and a two-class head; its
    cross entropy against `nsp` (1 = the two segments were swapped or unrelated) is added to the loss.
Not taken over: the separate output bias of the vocabulary projection.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List

import torch

from ..ops import functional as F
from ..parallel import mappings as M
from .base import Env, Op, OpInfo
from .gpt import GPT_LAYER_OPS
from .transformer_ops import (AttnDropoutOp, BiasActOp, BiasDropoutAddOp, ContextOp, DenseOp, EmbeddingOp,
                              LayerNormOp, MLPUpOp, QKVOp, ScoreOp, SoftmaxOp)


@dataclass
class BertConfig:
    num_layers: int = 24
    hidden: int = 1024
    heads: int = 16
    head_dim: int = 64
    ffn: int = 4096
    seq_length: int = 512
    vocab: int = 30592
    max_positions: int = 512
    num_tokentypes: int = 2
    binary_head: bool = True
    hidden_dropout: float = 0.1
    attention_dropout: float = 0.1
    layernorm_eps: float = 1e-5
    init_std: float = 0.02
    activation: int = F.ACT_GELU
    make_vocab_divisible_by: int = 128
    max_tp: int = 8

    @property
    def padded_vocab(self) -> int:
        m = self.make_vocab_divisible_by * self.max_tp
        return (self.vocab + m - 1) // m * m

    @property
    def output_init_std(self) -> float:
        return self.init_std / (2.0 * self.num_layers) ** 0.5


def bert_op_names(num_layers: int) -> List[str]:
    return ["encoder-embedding"] + GPT_LAYER_OPS * num_layers + ["final-layernorm", "bert-post-process"]


def bert_layer_of(index: int, num_layers: int) -> int:
    if index == 0 or index > 13 * num_layers:
        return -1
    return (index - 1) // 13


class BertEmbeddingOp(EmbeddingOp):
    """Word + position + token-type embeddings, then dropout (reference: Embedding with num_tokentypes = 2,
    runtime/megatron/model/language_model.py)."""
    reads = ("ids", "types")

    def __init__(self, info, env):
        super().__init__(info, env)
        self.reads = ("ids", "types")

    def declare(self):
        super().declare()
        c = self.env.cfg
        self.param_spec("tokentype_embeddings.weight", (c.num_tokentypes, c.hidden), "normal", std=c.init_std,
                        seed_key="tokentype_embeddings", shared_key="tokentype_embeddings")

    def forward(self, st):
        c = self.env.cfg
        ids = st["ids"]
        b, s = ids.shape
        pos = torch.arange(s, device=ids.device, dtype=torch.int64).repeat(b)
        W, P = self.p("word_embeddings.weight"), self.p("position_embeddings.weight")
        if self.pl.tp == 1:
            x = F.embedding(ids, pos, W, P, 0, 0.0, 0)
        else:
            x = F.embedding(ids, None, W, None, self.pl.tp_rank * self.v_local, 0.0, 0)
            x = M.reduce_from_group(x, self.tp_group)
            # positions are 0 .. s-1 in every sample: add the first s rows to each sample (no gather; the gradient of
            # a row is then a reduction over the batch, accumulated in fp32)
            x = (x.view(b, s, -1) + P[:s]).view(b * s, -1)
        types = st.get("types")
        if types is not None:
            # looked up in fp32: the gradient of a row is the sum over all tokens of that type, which bf16 would round
            # at every addition
            x = x + torch.nn.functional.embedding(types.reshape(-1), self.p("tokentype_embeddings.weight").float()).to(x.dtype)
        p_drop = c.hidden_dropout if self.env.training else 0.0
        st["x"] = F.dropout(x, p_drop, self.seed()) if p_drop > 0.0 else x


class BertPostOp(Op):
    """LM head (dense + GeLU + LayerNorm + tied vocabulary projection + masked cross entropy) and, with
    `binary_head`, pooler + two-class head + cross entropy (Megatron-LM's BertLMHead and BERT loss; the labels are
    the ones runtime/megatron/data/bert_dataset.py builds: `labels`, `loss_mask`, `is_random`)."""
    reads = ("x", "labels", "loss_mask", "nsp")
    writes = ("loss", "logits")

    def declare(self):
        c = self.env.cfg
        v = c.padded_vocab
        self.v_local = v // self.pl.tp
        h = c.hidden
        self.param_spec("word_embeddings.weight", (self.v_local, h), "normal", full_shape=(v, h), shard_dim=0,
                        std=c.init_std, seed_key="word_embeddings", shared_key="word_embeddings")
        self.param_spec("lm_head.dense.weight", (h, h), "normal", std=c.init_std)
        self.param_spec("lm_head.dense.bias", (h,), "zeros", weight_decay=False)
        self.param_spec("lm_head.layernorm.weight", (h,), "ones", weight_decay=False, fp32=True)
        self.param_spec("lm_head.layernorm.bias", (h,), "zeros", weight_decay=False, fp32=True)
        if c.binary_head:
            self.param_spec("pooler.dense.weight", (h, h), "normal", std=c.init_std)
            self.param_spec("pooler.dense.bias", (h,), "zeros", weight_decay=False)
            self.param_spec("binary_head.weight", (2, h), "normal", std=c.init_std)
            self.param_spec("binary_head.bias", (2,), "zeros", weight_decay=False)

    def forward(self, st):
        c = self.env.cfg
        x = st["x"]
        t = F.linear(x, self.p("lm_head.dense.weight"), self.p("lm_head.dense.bias"), act=F.ACT_GELU)
        t = F.layernorm(t, self.p("lm_head.layernorm.weight"), self.p("lm_head.layernorm.bias"), c.layernorm_eps)
        # the vocabulary projection is sharded over the tensor-parallel ranks: each rank's gradient of t covers its
        # shard only, and the identity-forward / all-reduce-backward mapping completes it BEFORE it reaches the
        # (replicated) transform parameters, whose gradients are then whole and equal on every rank
        t = M.copy_to_group(t, self.tp_group)
        if "labels" not in st:
            logits = F.linear(t, self.p("word_embeddings.weight"))
            st["logits"] = M.gather_from_group(logits, -1, self.tp_group)
            return
        labels = st["labels"]
        scale = st.get("loss_scale", 1.0)
        mask = st.get("loss_mask")
        if mask is None:
            weights, lm_scale = None, scale / labels.numel()
        else:
            m = mask.reshape(-1).float()
            weights, lm_scale = m / m.sum().clamp(min=1.0), scale
        safe = labels.clamp(min=0)                       # positions without a label carry -1 and a zero weight
        loss = F.lm_head_cross_entropy(t, self.p("word_embeddings.weight"), safe, weights,
                                       self.pl.tp_rank * self.v_local, lm_scale, self.tp_group)
        nsp = st.get("nsp")
        if c.binary_head and nsp is not None:
            b = labels.shape[0]
            first = x.view(b, -1, x.shape[-1])[:, 0].float()
            pooled = torch.tanh(first @ self.p("pooler.dense.weight").float().t() + self.p("pooler.dense.bias").float())
            two = pooled @ self.p("binary_head.weight").float().t() + self.p("binary_head.bias").float()
            keep = nsp >= 0                                # -1 = no sentence-order label for this sample
            per = torch.nn.functional.cross_entropy(two, nsp.clamp(min=0), reduction="none") * keep.float()
            loss = loss + per.sum() / keep.float().sum().clamp(min=1.0) * scale
        st["loss"] = loss


def build_bert_op(info: OpInfo, env: Env) -> Op:
    c = env.cfg
    n = info.name
    if n == "encoder-embedding":
        return BertEmbeddingOp(info, env)
    if n in ("enc-1st-layernorm", "enc-2nd-layernorm"):
        return LayerNormOp(info, env)
    if n == "final-layernorm":
        return LayerNormOp(info, env, keep_residual=False)
    if n == "enc-attention-qkv":
        return QKVOp(info, env)
    if n == "enc-attention-score":
        return ScoreOp(info, env, mode="full")
    if n == "enc-attention-softmax":
        return SoftmaxOp(info, env, mode="full")
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
    if n == "bert-post-process":
        return BertPostOp(info, env)
    raise KeyError(f"unknown BERT op {n}")


def bert_config_from_plan(d: dict, **overrides) -> BertConfig:
    heads = d["num_attention_heads"]
    cfg = BertConfig(num_layers=d["num_layers"], hidden=d["hidden_size"], heads=heads,
                     head_dim=d.get("kv_channels", d["hidden_size"] // heads),
                     ffn=d.get("ffn_hidden_size", 4 * d["hidden_size"]), seq_length=d["seq_length"],
                     max_positions=d.get("max_position_embeddings", d["seq_length"]), vocab=d.get("vocab_size", 30592),
                     binary_head=bool(d.get("binary_head", True)))
    for k, v in overrides.items():
        setattr(cfg, k, v)
    return cfg
