"""BERT, ViT and the inverse-cloze biencoder on the GPU: three training steps of small plans through the native
kernels (flash attention with padding lengths, GEMM epilogues, LayerNorm, dropout), finite losses, clean status word."""
import math

import pytest
import torch

from helpers import tiny_bert_plan, tiny_ict_plan, tiny_vit_plan
from superscaler_b200.data import synthetic as syn
from superscaler_b200.ops import native

pytestmark = pytest.mark.gpu
KW = dict(layers=2, hidden=128, heads=2, head_dim=64, global_bs=8, micro_bs=4)


def _ict_batch(seed):
    b = syn.bert_batch(8, 64, 512, seed=seed)
    ids = b["ids"]
    ids[1::2] = ids[0::2]
    return {"ids": ids, "types": torch.zeros_like(ids), "enc_lens": b["enc_lens"],
            "labels": torch.arange(4).repeat_interleave(2)}


@pytest.mark.parametrize("name", ["bert", "vit", "ict"])
def test_three_training_steps(name):
    from superscaler_b200.runtime.trainer import Trainer
    plan, batch = {
        "bert": (tiny_bert_plan(seq=64, vocab=512, **KW), lambda s: syn.bert_batch(8, 64, 512, seed=s)),
        "vit": (tiny_vit_plan(image_size=64, patch=16, num_classes=10, **KW), lambda s: syn.resnet_batch(8, 64, 10, seed=s)),
        "ict": (tiny_ict_plan(seq=64, vocab=512, **KW), _ict_batch),
    }[name]
    t = Trainer(plan, rank=0, world_size=1)
    losses = [t.loss_value(t.train_step(batch(1))) for _ in range(3)]
    torch.cuda.synchronize()
    assert all(math.isfinite(v) for v in losses), losses
    assert native.check_status() == 0
    expect = {"bert": math.log(512) + math.log(2), "vit": math.log(10), "ict": math.log(4)}[name]
    assert abs(losses[0] - expect) < 1.5, (losses, expect)       # untrained: near the entropy of a uniform guess
