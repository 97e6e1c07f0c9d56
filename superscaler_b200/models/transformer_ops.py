"""Transformer operators (GPT and T5 op lists) on the sm_100a kernels.

One class per op name of the reference's flat op list (runtime/megatron/model/flex_ops.py:89-222), so a
plan can place, shard and recompute every op individually; `fuse_ops` then collapses co-located
neighbours into the fused kernels (flash attention, GEMM + bias-GeLU, GEMM + bias-dropout-residual).

Activation layout: [tokens, features] bf16, tokens batch-major (row = b * s + s_idx).  A data-parallel
split is therefore a contiguous row split, a tensor-parallel split of the hidden dimension a column
split.  Tensor-parallel algorithms: algo 0 is the Megatron pairing (QKV / MLP-1 column-parallel,
dense / MLP-2 row-parallel); algo 1 swaps the roles (flex_ops.py:483-538,1027-1056).
"""
from __future__ import annotations

import math

import torch

from ..ops import functional as F
from ..parallel import mappings as M
from .base import Op


def _prefix(name: str) -> str:
    return name.split("-")[0]  # "enc" / "dec" / "encoder" ...


class EmbeddingOp(Op):
    """Vocab-parallel word embedding + learned position embedding + dropout.
    Reference: Embedding, runtime/megatron/model/flex_ops.py:229-380."""
    reads = ("ids",)
    writes = ("x",)

    def __init__(self, info, env, ids_key="ids", seq_attr="seq_length"):
        super().__init__(info, env)
        self.ids_key = ids_key
        self.seq = getattr(env.cfg, seq_attr)
        self.reads = (ids_key,)

    def declare(self):
        c = self.env.cfg
        v = c.padded_vocab
        self.v_local = v // self.pl.tp
        self.param_spec("word_embeddings.weight", (self.v_local, c.hidden), "normal", full_shape=(v, c.hidden),
                        shard_dim=0, std=c.init_std, seed_key="word_embeddings", shared_key="word_embeddings")
        self.param_spec("position_embeddings.weight", (c.max_positions, c.hidden), "normal", std=c.init_std,
                        seed_key="position_embeddings", shared_key="position_embeddings")

    def forward(self, st):
        c = self.env.cfg
        ids = st[self.ids_key]
        b, s = ids.shape
        pos = torch.arange(s, device=ids.device, dtype=torch.int64).repeat(b)
        W, P = self.p("word_embeddings.weight"), self.p("position_embeddings.weight")
        p_drop = c.hidden_dropout if self.env.training else 0.0
        if self.pl.tp == 1:
            st["x"] = F.embedding(ids, pos, W, P, 0, p_drop, self.seed())
        else:
            x = F.embedding(ids, None, W, None, self.pl.tp_rank * self.v_local, 0.0, 0)
            x = M.reduce_from_group(x, self.tp_group)
            # positions are 0 .. s-1 in every sample: add the first s rows to each sample (no gather; the gradient of
            # a row is then a reduction over the batch, accumulated in fp32)
            x = (x.view(b, s, -1) + P[:s]).view(b * s, -1)
            st["x"] = F.dropout(x, p_drop, self.seed())


class LayerNormOp(Op):
    """LayerNorm; keeps its input as the residual for the next residual add.
    Reference: ParallelLayerNormOp, flex_ops.py:382-473."""
    reads = ("x",)
    writes = ("x", "residual")

    def __init__(self, info, env, keep_residual=True):
        super().__init__(info, env)
        self.keep_residual = keep_residual
        if not keep_residual:
            self.writes = ("x",)

    def declare(self):
        h = self.env.cfg.hidden
        self.param_spec("layernorm.weight", (h,), "ones", weight_decay=False, fp32=True)
        self.param_spec("layernorm.bias", (h,), "zeros", weight_decay=False, fp32=True)

    def forward(self, st):
        x = st["x"]
        if self.keep_residual:
            st["x"], st["residual"] = F.layernorm_keep_input(x, self.p("layernorm.weight"), self.p("layernorm.bias"),
                                                             self.env.cfg.layernorm_eps)
        else:
            st["x"] = F.layernorm(x, self.p("layernorm.weight"), self.p("layernorm.bias"), self.env.cfg.layernorm_eps)


class QKVOp(Op):
    """Fused query/key/value projection.  Output columns are [Q heads | K heads | V heads] of the local heads.
    kind: "self" (one GEMM on x), "cross" (Q from x, K/V from the encoder output).
    Reference: ParallelQKVOp, flex_ops.py:475-709."""
    reads = ("x",)
    writes = ("x",)

    def __init__(self, info, env, kind="self"):
        super().__init__(info, env)
        self.kind = kind
        if kind == "cross":
            self.reads = ("x", "enc_out")
            self.writes = ("x", "kv")

    def declare(self):
        c = self.env.cfg
        h, proj, tp = c.hidden, c.heads * c.head_dim, self.pl.tp
        if self.info.algo == 0:
            if self.kind == "self":
                self.param_spec("query_key_value.weight", (3, proj // tp, h), "normal", full_shape=(3, proj, h),
                                shard_dim=1, std=c.init_std)
                self.param_spec("query_key_value.bias", (3, proj // tp), "zeros", weight_decay=False,
                                full_shape=(3, proj), shard_dim=1)
            else:
                self.param_spec("query.weight", (proj // tp, h), "normal", full_shape=(proj, h), shard_dim=0,
                                std=c.init_std)
                self.param_spec("query.bias", (proj // tp,), "zeros", weight_decay=False, full_shape=(proj,),
                                shard_dim=0)
                self.param_spec("key_value.weight", (2, proj // tp, h), "normal", full_shape=(2, proj, h),
                                shard_dim=1, std=c.init_std)
                self.param_spec("key_value.bias", (2, proj // tp), "zeros", weight_decay=False,
                                full_shape=(2, proj), shard_dim=1)
        else:
            assert self.kind == "self", "algo 1 exists for self-attention QKV only"
            self.param_spec("query_key_value.weight", (3 * proj, h // tp), "normal", full_shape=(3 * proj, h),
                            shard_dim=1, std=c.init_std)
            self.param_spec("query_key_value.bias", (3 * proj,), "zeros", weight_decay=False)

    def accepts_dealt_out_rows(self) -> bool:
        return self.info.algo == 0 and self.kind == "self"

    def forward(self, st):
        x = st["x"]
        if st.pop("_x_rows_dealt_out", False):
            w = self.p("query_key_value.weight")
            st["x"] = F.gathered_column_linear_fused(x, w.view(-1, w.shape[-1]), self.p("query_key_value.bias").view(-1),
                                                     F.ACT_NONE, self.tpctx())
        elif self.info.algo == 0 and self.kind == "self" and self.tpctx() is not None:
            w = self.p("query_key_value.weight")
            st["x"] = F.column_parallel_linear_fused(x, w.view(-1, w.shape[-1]), self.p("query_key_value.bias").view(-1),
                                                     F.ACT_NONE, self.tpctx())
        elif self.info.algo == 0:
            xin = M.copy_to_group(x, self.tp_group)
            if self.kind == "self":
                w = self.p("query_key_value.weight")
                st["x"] = F.linear(xin, w.view(-1, w.shape[-1]), self.p("query_key_value.bias").view(-1))
            else:
                st["x"] = F.linear(xin, self.p("query.weight"), self.p("query.bias"))
                w = self.p("key_value.weight")
                enc = M.copy_to_group(st["enc_out"], self.tp_group)
                st["kv"] = F.linear(enc, w.view(-1, w.shape[-1]), self.p("key_value.bias").view(-1))
        else:
            # row-parallel: the input arrives split along the hidden dimension, partial outputs are summed
            y = F.linear(x, self.p("query_key_value.weight"), None)
            y = M.reduce_from_group(y, self.tp_group)
            st["x"] = F.bias_dropout_add(y, self.p("query_key_value.bias"), torch.zeros_like(y), 0.0, 0)


class _AttnDims:
    def dims(self, st):
        c = self.env.cfg
        nh = c.heads // self.pl.tp
        return nh, c.head_dim


class _RelativeBias:
    """T5 relative-position bias of a self-attention op: one [heads, buckets] table per stack (encoder looks both
    ways, decoder backwards only), declared by the score op and shared by all layers of the stack."""

    def uses_relative_bias(self) -> bool:
        return bool(getattr(self.env.cfg, "relative_position_bias", False)) and self.mode != "cross"

    def declare_relative_bias(self) -> None:
        if not self.uses_relative_bias():
            return
        c = self.env.cfg
        stack = "dec" if self.mode == "causal" else "enc"
        self.param_spec("relative_attention_bias.weight", (c.heads // self.pl.tp, c.relative_attention_num_buckets),
                        "normal", full_shape=(c.heads, c.relative_attention_num_buckets), shard_dim=0, std=c.init_std,
                        weight_decay=False, fp32=True, seed_key=f"{stack}_relative_attention_bias",
                        shared_key=f"{stack}_relative_attention_bias")

    def relative_bias(self, sq: int, sk: int) -> torch.Tensor:
        """[local heads, sq, sk] fp32 (reference path; a kernel takes the distance table instead)."""
        from .relative_position import bias_from_table, distance_table
        c = self.env.cfg
        return bias_from_table(self.relative_bias_table(sq, sk), sq, sk)

    def relative_bias_table(self, sq: int, sk: int) -> torch.Tensor:
        """[local heads, sq + sk - 1] fp32, differentiable: entry d - (sq - 1) ... the bias of distance key - query = d.
        This is what the flash-attention kernels take (the bias depends on the distance alone)."""
        from .relative_position import distance_table
        c = self.env.cfg
        w = self.p("relative_attention_bias.weight")
        return distance_table(w.float(), sq, sk, self.mode != "causal", c.relative_attention_num_buckets,
                              c.relative_attention_max_distance)


def key_lengths(op: Op, st):
    """Number of real (unpadded) encoder tokens of every sample this op sees, or None: its own data-parallel share
    of the micro-batch's lengths when the trainer supplied them all (`enc_lens_all`), else `enc_lens` as given."""
    full = st.get("enc_lens_all")
    if full is None:
        return st.get("enc_lens")
    return full[op.pl.dp_rank * op.local_bs:(op.pl.dp_rank + 1) * op.local_bs]


class AttentionCoreOp(Op, _AttnDims, _RelativeBias):
    """score + softmax + dropout + context as ONE flash-attention kernel (the fused form of the four
    reference ops flex_ops.py:711-1015).  mode: "causal" | "full" | "cross"."""
    reads = ("x",)
    writes = ("x",)

    def __init__(self, info, env, mode="causal", sq_attr="seq_length", sk_attr="seq_length"):
        super().__init__(info, env)
        self.mode = mode
        self.sq, self.sk = getattr(env.cfg, sq_attr), getattr(env.cfg, sk_attr)
        if mode == "cross":
            self.reads = ("x", "kv")

    def forward(self, st):
        c = self.env.cfg
        nh, hd = self.dims(st)
        w = nh * hd
        p_drop = c.attention_dropout if self.env.training else 0.0
        x = st["x"]
        b = x.shape[0] // self.sq
        scale = 1.0 / math.sqrt(hd)
        if self.uses_relative_bias() and x.is_cuda:
            st["x"] = F.flash_attention(x, x, x, b, nh, self.sq, self.sq, hd, cols=(0, w, 2 * w), scale=scale,
                                        causal=self.mode == "causal",
                                        kv_lens=key_lengths(self, st) if self.mode == "full" else None,
                                        dropout_p=p_drop, seed=self.seed(sharded=True),
                                        bias_table=self.relative_bias_table(self.sq, self.sq))
        elif self.uses_relative_bias():
            st["x"] = F.attention_with_bias(x, b, nh, self.sq, hd, scale, self.mode == "causal",
                                            key_lengths(self, st) if self.mode == "full" else None,
                                            self.relative_bias(self.sq, self.sq), p_drop)
        elif self.mode == "cross":
            kv = st["kv"]
            st["x"] = F.flash_attention(x, kv, kv, b, nh, self.sq, self.sk, hd, cols=(0, 0, w), scale=scale,
                                        causal=False, kv_lens=key_lengths(self, st), dropout_p=p_drop,
                                        seed=self.seed(sharded=True))
        else:
            st["x"] = F.flash_attention(x, x, x, b, nh, self.sq, self.sq, hd, cols=(0, w, 2 * w), scale=scale,
                                        causal=self.mode == "causal",
                                        kv_lens=key_lengths(self, st) if self.mode == "full" else None,
                                        dropout_p=p_drop, seed=self.seed(sharded=True))


class DenseOp(Op):
    """Output projection of attention or second MLP GEMM without its bias (the bias rides to the following
    dropout op as "bias").  algo 0: row-parallel (input split along features, output all-reduced);
    algo 1: column-parallel.  Reference: ParallelGEMM, flex_ops.py:1022-1124."""
    reads = ("x",)
    writes = ("x", "bias")

    def __init__(self, info, env, key="dense", in_features=None, out_features=None):
        super().__init__(info, env)
        self.key, self.fin, self.fout = key, in_features, out_features

    def declare(self):
        c, tp = self.env.cfg, self.pl.tp
        if self.info.algo == 0:
            self.param_spec(f"{self.key}.weight", (self.fout, self.fin // tp), "normal", full_shape=(self.fout, self.fin),
                            shard_dim=1, std=c.output_init_std)
            self.param_spec(f"{self.key}.bias", (self.fout,), "zeros", weight_decay=False)
        else:
            self.param_spec(f"{self.key}.weight", (self.fout // tp, self.fin), "normal", full_shape=(self.fout, self.fin),
                            shard_dim=0, std=c.output_init_std)
            self.param_spec(f"{self.key}.bias", (self.fout // tp,), "zeros", full_shape=(self.fout,), shard_dim=0,
                            weight_decay=False)

    def forward(self, st):
        x = st["x"]
        if self.info.algo == 0:
            y = F.linear(x, self.p(f"{self.key}.weight"), None)
            st["x"] = M.reduce_from_group(y, self.tp_group)
        else:
            st["x"] = F.linear(M.copy_to_group(x, self.tp_group), self.p(f"{self.key}.weight"), None)
        st["bias"] = self.p(f"{self.key}.bias")


class BiasDropoutAddOp(Op):
    """x = residual + dropout(x + bias).  Reference: ParallelDropoutOp, flex_ops.py:1126-1227."""
    reads = ("x", "bias", "residual")
    writes = ("x",)

    def forward(self, st):
        p_drop = self.env.cfg.hidden_dropout if self.env.training else 0.0
        st["x"] = F.bias_dropout_add(st["x"], st.pop("bias"), st.pop("residual"), p_drop, self.seed())


class MLPUpOp(Op):
    """First MLP GEMM without bias (bias rides to the activation op).  algo 0 column-parallel, algo 1 row-parallel."""
    reads = ("x",)
    writes = ("x", "bias")

    def declare(self):
        c, tp = self.env.cfg, self.pl.tp
        if self.info.algo == 0:
            self.param_spec("dense_h_to_4h.weight", (c.ffn // tp, c.hidden), "normal", full_shape=(c.ffn, c.hidden),
                            shard_dim=0, std=c.init_std)
            self.param_spec("dense_h_to_4h.bias", (c.ffn // tp,), "zeros", full_shape=(c.ffn,), shard_dim=0,
                            weight_decay=False)
        else:
            self.param_spec("dense_h_to_4h.weight", (c.ffn, c.hidden // tp), "normal", full_shape=(c.ffn, c.hidden),
                            shard_dim=1, std=c.init_std)
            self.param_spec("dense_h_to_4h.bias", (c.ffn,), "zeros", weight_decay=False)

    def forward(self, st):
        x = st["x"]
        if self.info.algo == 0:
            st["x"] = F.linear(M.copy_to_group(x, self.tp_group), self.p("dense_h_to_4h.weight"), None)
        else:
            st["x"] = M.reduce_from_group(F.linear(x, self.p("dense_h_to_4h.weight"), None), self.tp_group)
        st["bias"] = self.p("dense_h_to_4h.bias")


class BiasActOp(Op):
    """x = act(x + bias).  Reference: ParallelMlpGeLUOp, flex_ops.py:1229-1281."""
    reads = ("x", "bias")
    writes = ("x",)

    def forward(self, st):
        st["x"] = F.bias_act(st["x"], st.pop("bias"), self.env.cfg.activation)


class LMHeadLossOp(Op):
    """Tied-embedding LM head + vocab-parallel cross entropy -> scalar loss for this micro-batch.
    Reference: GPTPostProcess / T5PostProcess, flex_ops.py:1283-1419."""
    reads = ("x", "labels", "loss_mask")
    writes = ("loss", "logits")

    def declare(self):
        c = self.env.cfg
        v = c.padded_vocab
        self.v_local = v // self.pl.tp
        self.param_spec("word_embeddings.weight", (self.v_local, c.hidden), "normal", full_shape=(v, c.hidden),
                        shard_dim=0, std=c.init_std, seed_key="word_embeddings", shared_key="word_embeddings")

    def forward(self, st):
        x = M.copy_to_group(st["x"], self.tp_group)
        if "labels" not in st:
            # inference: full-vocabulary logits [tokens, padded vocab] instead of a loss (text generation, scoring)
            logits = F.linear(x, self.p("word_embeddings.weight"))
            st["logits"] = M.gather_from_group(logits, -1, self.tp_group)
            return
        labels = st["labels"]
        mask = st.get("loss_mask")
        scale = st.get("loss_scale", 1.0)
        if mask is None:
            weights, scale = None, scale / labels.numel()
        else:
            # masked mean as the reference's loss_func (runtime/pretrain_gpt.py:64-72, pretrain_t5.py:88-99):
            # sum(loss * mask) / mask.sum() over this rank's rows; the division rides in the per-row weights so
            # that no count has to be read back to the host
            m = mask.reshape(-1).float()
            weights = m / m.sum().clamp(min=1.0)
        st["loss"] = F.lm_head_cross_entropy(x, self.p("word_embeddings.weight"), labels, weights,
                                             self.pl.tp_rank * self.v_local, scale, self.tp_group)


# ------------------------------------------------------------------------------------------------
# Unfused attention pieces (only used when a plan separates them; slow path, one GEMM per head)
# ------------------------------------------------------------------------------------------------
class ScoreOp(Op, _AttnDims, _RelativeBias):
    """scores[b, h] = Q K^T (unscaled; the softmax op applies the scale); keeps V as "value"."""
    reads = ("x",)
    writes = ("x", "value")

    def __init__(self, info, env, mode="causal", sq_attr="seq_length", sk_attr="seq_length"):
        super().__init__(info, env)
        self.mode = mode
        self.sq, self.sk = getattr(env.cfg, sq_attr), getattr(env.cfg, sk_attr)
        if mode == "cross":
            self.reads = ("x", "kv")

    def declare(self):
        self.declare_relative_bias()

    def forward(self, st):
        nh, hd = self.dims(st)
        w = nh * hd
        x = st["x"]
        b = x.shape[0] // self.sq
        if self.mode == "cross":
            q, k, v = x, st["kv"][:, :w], st.pop("kv")[:, w:]
        else:
            q, k, v = x[:, :w], x[:, w:2 * w], x[:, 2 * w:]
        scores = []
        for bi in range(b):
            for hi in range(nh):
                qq = q[bi * self.sq:(bi + 1) * self.sq, hi * hd:(hi + 1) * hd]
                kk = k[bi * self.sk:(bi + 1) * self.sk, hi * hd:(hi + 1) * hd]
                scores.append(F.linear(qq, kk))
        st["x"] = torch.stack(scores).view(b, nh, self.sq, self.sk)
        if self.uses_relative_bias():
            # the softmax op multiplies by 1 / sqrt(head_dim): the bias is added pre-divided so that it arrives whole
            st["x"] = st["x"] + (self.relative_bias(self.sq, self.sk) * math.sqrt(hd)).to(st["x"].dtype)
        st["value"] = v


class SoftmaxOp(Op, _AttnDims):
    reads = ("x",)
    writes = ("x",)

    def __init__(self, info, env, mode="causal"):
        super().__init__(info, env)
        self.mode = mode

    def forward(self, st):
        scale = 1.0 / math.sqrt(self.env.cfg.head_dim)
        x = st["x"]
        lens = key_lengths(self, st) if self.mode != "causal" else None
        if lens is None:
            st["x"] = F.scaled_softmax(x, scale, 1 if self.mode == "causal" else 0)
            return
        # padded keys (the encoder's, also for the decoder's cross attention) get no weight, as in the one-kernel
        # attention, which takes the same lengths as kv_lens
        b, _, sq, sk = x.shape
        beyond = torch.arange(sk, device=x.device)[None, :] >= lens.to(x.device).view(b, 1)
        mask = beyond.view(b, 1, 1, sk).expand(b, 1, sq, sk).to(torch.uint8).contiguous()
        st["x"] = F.scaled_softmax(x, scale, 2, mask)


class AttnDropoutOp(Op):
    reads = ("x",)
    writes = ("x",)

    def forward(self, st):
        p_drop = self.env.cfg.attention_dropout if self.env.training else 0.0
        x = st["x"]
        st["x"] = F.dropout(x.reshape(-1, x.shape[-1]), p_drop, self.seed(sharded=True)).view_as(x)


class ContextOp(Op, _AttnDims):
    reads = ("x", "value")
    writes = ("x",)

    def forward(self, st):
        nh, hd = self.dims(st)
        probs, v = st["x"], st.pop("value")
        b, _, sq, sk = probs.shape
        out = torch.empty(b * sq, nh * hd, dtype=probs.dtype, device=probs.device)
        cols = []
        for bi in range(b):
            row = []
            for hi in range(nh):
                vv = v[bi * sk:(bi + 1) * sk, hi * hd:(hi + 1) * hd]
                row.append(F.linear(probs[bi, hi], vv.t().contiguous()))
            cols.append(torch.cat(row, dim=1))
        st["x"] = torch.cat(cols, dim=0)
