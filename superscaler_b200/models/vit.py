"""Vision transformer (image classification) as a flat op list: `vit-embedding` (patches -> linear projection, class
token, learned positions), 13 ops per layer (the encoder layer names shared with GPT / T5 / BERT), `final-layernorm`,
`vit-post-process` (MLP head on the class token + cross entropy).

The reference's tree holds this model's flags (`_add_vit_args`, runtime/megatron/arguments.py:760-772: --num-classes,
--img-dim, --patch-dim) and its data pipeline (runtime/megatron/data/vit_dataset.py, autoaugment.py), inherited from
Megatron-LM, but not the model file they were written for; the model here follows Megatron-LM's vision transformer
(patch projection, class token, learned positions, MLP head) and, unlike it, runs from a plan.  Images arrive channels-last [b, H, W, 3], as for the
Wide-ResNet; a patch is flattened in (row, column, channel) order.  seq_length = (image_size / patch)^2 + 1.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List

import torch

from ..ops import functional as F
from .base import Env, Op, OpInfo
from .gpt import GPT_LAYER_OPS
from .transformer_ops import (AttnDropoutOp, BiasActOp, BiasDropoutAddOp, ContextOp, DenseOp, LayerNormOp, MLPUpOp,
                              QKVOp, ScoreOp, SoftmaxOp)


@dataclass
class VitConfig:
    num_layers: int = 12
    hidden: int = 768
    heads: int = 12
    head_dim: int = 64
    ffn: int = 3072
    image_size: int = 224
    patch: int = 16
    num_classes: int = 1000
    hidden_dropout: float = 0.1
    attention_dropout: float = 0.1
    layernorm_eps: float = 1e-5
    init_std: float = 0.02
    activation: int = F.ACT_GELU
    max_tp: int = 8

    @property
    def num_patches(self) -> int:
        return (self.image_size // self.patch) ** 2

    @property
    def seq_length(self) -> int:
        return self.num_patches + 1

    @property
    def output_init_std(self) -> float:
        return self.init_std / (2.0 * self.num_layers) ** 0.5


def vit_op_names(num_layers: int) -> List[str]:
    return ["vit-embedding"] + GPT_LAYER_OPS * num_layers + ["final-layernorm", "vit-post-process"]


def vit_layer_of(index: int, num_layers: int) -> int:
    if index == 0 or index > 13 * num_layers:
        return -1
    return (index - 1) // 13


class VitEmbeddingOp(Op):
    """Patches -> linear projection; a learned class token in front; learned position embeddings; dropout
    (Megatron-LM's VitModel.forward; patch and image sizes as --patch-dim / --img-dim of
    runtime/megatron/arguments.py:760-772)."""
    reads = ("images",)
    writes = ("x",)

    def declare(self):
        c = self.env.cfg
        k = c.patch * c.patch * 3
        self.param_spec("linear_encoder.weight", (c.hidden, k), "normal", std=c.init_std)
        self.param_spec("linear_encoder.bias", (c.hidden,), "zeros", weight_decay=False)
        self.param_spec("cls_token", (1, c.hidden), "zeros", weight_decay=False)
        self.param_spec("position_embeddings.weight", (c.seq_length, c.hidden), "normal", std=c.init_std)

    def forward(self, st):
        c = self.env.cfg
        img = st["images"]
        b, H, W, ch = img.shape
        p, g = c.patch, c.image_size // c.patch
        assert H == c.image_size and W == c.image_size and ch == 3, f"images must be [b, {c.image_size}, {c.image_size}, 3]"
        patches = img.view(b, g, p, g, p, ch).permute(0, 1, 3, 2, 4, 5).reshape(b * g * g, p * p * ch).contiguous()
        x = F.linear(patches, self.p("linear_encoder.weight"), self.p("linear_encoder.bias"))
        x = torch.cat([self.p("cls_token").to(x.dtype).expand(b, 1, c.hidden), x.view(b, g * g, c.hidden)], dim=1)
        x = (x + self.p("position_embeddings.weight").to(x.dtype)[None]).reshape(b * c.seq_length, c.hidden)
        p_drop = c.hidden_dropout if self.env.training else 0.0
        st["x"] = F.dropout(x.contiguous(), p_drop, self.seed()) if p_drop > 0.0 else x.contiguous()


class VitPostOp(Op):
    """Class-token head: dense + tanh + dense -> class logits, cross entropy (Megatron-LM's VitMlpHead)."""
    reads = ("x", "labels")
    writes = ("loss", "logits")

    def declare(self):
        c = self.env.cfg
        self.param_spec("head.dense_in.weight", (c.hidden, c.hidden), "normal", std=c.init_std)
        self.param_spec("head.dense_in.bias", (c.hidden,), "zeros", weight_decay=False)
        self.param_spec("head.dense_out.weight", (c.num_classes, c.hidden), "normal", std=c.init_std)
        self.param_spec("head.dense_out.bias", (c.num_classes,), "zeros", weight_decay=False)

    def forward(self, st):
        c = self.env.cfg
        x = st["x"]
        b = x.shape[0] // c.seq_length
        first = x.view(b, c.seq_length, c.hidden)[:, 0].float()
        t = torch.tanh(first @ self.p("head.dense_in.weight").float().t() + self.p("head.dense_in.bias").float())
        logits = t @ self.p("head.dense_out.weight").float().t() + self.p("head.dense_out.bias").float()
        if "labels" not in st:
            st["logits"] = logits
            return
        scale = st.get("loss_scale", 1.0)
        loss = torch.nn.functional.cross_entropy(logits, st["labels"]) * scale
        if not self.env.training:         # evaluation: [loss, share of samples whose best class is the label]
            loss = torch.stack([loss, (logits.argmax(-1) == st["labels"]).float().mean() * scale])
        st["loss"] = loss


def build_vit_op(info: OpInfo, env: Env) -> Op:
    c = env.cfg
    n = info.name
    if n == "vit-embedding":
        return VitEmbeddingOp(info, env)
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
    if n == "vit-post-process":
        return VitPostOp(info, env)
    raise KeyError(f"unknown ViT op {n}")


def vit_config_from_plan(d: dict, **overrides) -> VitConfig:
    heads = d["num_attention_heads"]
    cfg = VitConfig(num_layers=d["num_layers"], hidden=d["hidden_size"], heads=heads,
                    head_dim=d.get("kv_channels", d["hidden_size"] // heads),
                    ffn=d.get("ffn_hidden_size", 4 * d["hidden_size"]), image_size=d.get("image_size", 224),
                    patch=d.get("patch_dim", 16), num_classes=d.get("num_classes", 1000))
    for k, v in overrides.items():
        setattr(cfg, k, v)
    return cfg
