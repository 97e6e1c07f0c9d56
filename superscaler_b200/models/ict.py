"""Inverse-cloze-task biencoder (the retriever pre-training of REALM / ORQA) as an op-list model: a BERT encoder
embeds queries and evidence blocks, and every query has to pick its own block among the blocks of the batch.

What the reference's tree holds of this model: its flags (`_add_biencoder_args`, runtime/megatron/arguments.py:703-740:
--biencoder-projection-dim, --biencoder-shared-query-context-model, --titles-data-path, --query-in-block-prob,
--retriever-score-scaling), its data (runtime/megatron/data/ict_dataset.py, biencoder_dataset_utils.py) and the index
builder (runtime/megatron/indexer.py, which imports a `megatron.model.biencoder_model` the tree does not contain).
The model itself follows Megatron-LM's biencoder, which those files were written for: a BERT encoder, the [CLS]
state, an optional linear projection, in-batch softmax over query x block scores, optionally divided by
sqrt(hidden).  Built here: the SHARED-tower variant.  Queries and blocks travel as ONE batch of 2 b
sequences, row 2 i = query i and row 2 i + 1 = its block, so a data-parallel split of the rows keeps pairs together
and the encoder runs once over both; the negatives of a query are the other blocks of the micro-batch on ALL
data-parallel ranks (the embeddings are all-gathered over the data-parallel group before the scores are taken).  The op list is BERT's with `ict-post-process` at the end.

Without labels in the state (inference) the last op leaves the projected embedding of every sequence in
`st["logits"]`; `Trainer.embed` returns it, which is the embedder `data.retrieval.build_index` takes.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List

import torch

from ..parallel import mappings as M
from .base import Env, Op, OpInfo
from .bert import BertConfig, bert_config_from_plan, build_bert_op
from .gpt import GPT_LAYER_OPS


@dataclass
class IctConfig(BertConfig):
    projection_dim: int = 128          # 0 = use the pooled hidden state itself
    score_scaling: bool = False        # divide the scores by sqrt(hidden)
    binary_head: bool = False


def ict_op_names(num_layers: int) -> List[str]:
    return ["encoder-embedding"] + GPT_LAYER_OPS * num_layers + ["final-layernorm", "ict-post-process"]


def ict_layer_of(index: int, num_layers: int) -> int:
    if index == 0 or index > 13 * num_layers:
        return -1
    return (index - 1) // 13


class IctPostOp(Op):
    """[CLS] state -> (optional) linear projection -> in-batch retrieval loss."""
    reads = ("x", "labels")
    writes = ("loss", "logits")

    def declare(self):
        c = self.env.cfg
        if c.projection_dim > 0:
            self.param_spec("projection_enc.weight", (c.projection_dim, c.hidden), "normal", std=c.init_std)
            self.param_spec("projection_enc.bias", (c.projection_dim,), "zeros", weight_decay=False)

    def forward(self, st):
        c = self.env.cfg
        x = st["x"]
        n = x.shape[0] // c.seq_length
        pooled = x.view(n, c.seq_length, c.hidden)[:, 0].float()
        if c.projection_dim > 0:
            pooled = pooled @ self.p("projection_enc.weight").float().t() + self.p("projection_enc.bias").float()
        if "labels" not in st:
            st["logits"] = pooled
            return
        assert n % 2 == 0, "the inverse-cloze batch holds (query, block) pairs"
        dp = self.pl.dp
        if dp > 1:
            # every query is scored against the blocks of ALL data-parallel ranks (rows arrive in rank order, pairs
            # stay adjacent).  All ranks then hold the same loss, and the gradient averaging over the ranks would
            # count each embedding's contribution 1 / dp times: the factor dp on the way back makes the averaged
            # gradient the gradient of the one global loss
            pooled = pooled.detach() + dp * (pooled - pooled.detach())
            pooled = M.gather_from_group(pooled, 0, self.dp_group)
            n = pooled.shape[0]
        q, blocks = pooled[0::2], pooled[1::2]
        scores = q @ blocks.t()
        if c.score_scaling:
            scores = scores / (c.hidden ** 0.5)
        target = torch.arange(n // 2, device=scores.device)
        st["loss"] = torch.nn.functional.cross_entropy(scores, target) * st.get("loss_scale", 1.0)


def build_ict_op(info: OpInfo, env: Env) -> Op:
    if info.name == "ict-post-process":
        return IctPostOp(info, env)
    return build_bert_op(info, env)


def ict_config_from_plan(d: dict, **overrides) -> IctConfig:
    b = bert_config_from_plan(d)
    cfg = IctConfig(**{k: getattr(b, k) for k in BertConfig.__dataclass_fields__})
    cfg.binary_head = False
    cfg.projection_dim = int(d.get("biencoder_projection_dim", 128))
    cfg.score_scaling = bool(d.get("retriever_score_scaling", False))
    for k, v in overrides.items():
        setattr(cfg, k, v)
    return cfg


def ict_batch_of(dataset, indices) -> dict:
    """(query, block) pairs of an `InverseClozeDataset`, interleaved: ids / token types / real lengths of 2 n
    sequences, and `labels` = the pair index of every sequence (the loss only needs their presence)."""
    import numpy as np
    rows = [dataset[int(i) % len(dataset)] for i in indices]
    ids = np.stack([t for r in rows for t in (r["query_tokens"], r["block_tokens"])])
    lens = np.asarray([int(m.sum()) for r in rows for m in (r["query_pad_mask"], r["block_pad_mask"])], dtype=np.int32)
    out = {"ids": torch.from_numpy(ids), "types": torch.zeros(ids.shape, dtype=torch.int64),
           "enc_lens": torch.from_numpy(lens), "labels": torch.arange(len(rows)).repeat_interleave(2)}
    return {k: v.pin_memory() for k, v in out.items()} if torch.cuda.is_available() else out
