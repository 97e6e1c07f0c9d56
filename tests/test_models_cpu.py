"""T5 and Wide-ResNet op lists train on CPU; fused, unfused and recomputed executions agree."""
import torch

from superscaler_b200.data.synthetic import resnet_batch, t5_batch
from superscaler_b200.models.gpt import gpt_op_names
from superscaler_b200.models.resnet import ResNetConfig, resnet_op_names
from superscaler_b200.models.static_info import live_keys_before, op_io
from superscaler_b200.models.t5 import t5_op_names
from superscaler_b200.runtime.trainer import Trainer

from helpers import tiny_resnet_plan, tiny_t5_plan


def test_op_counts_match_the_reference_models():
    assert len(gpt_op_names(24)) == 315
    assert len(t5_op_names(24)) == 821
    assert len(resnet_op_names(ResNetConfig())) == 134
    for name in gpt_op_names(1) + t5_op_names(1) + resnet_op_names(ResNetConfig()):
        op_io(name)  # every op has static read / write information


def test_boundary_liveness():
    names = gpt_op_names(2)
    assert live_keys_before(names, 1) == ["x"]
    assert set(live_keys_before(names, names.index("enc-attention-qkv"))) == {"x", "residual"}
    assert set(live_keys_before(names, names.index("enc-post-attention-dropout"))) == {"x", "bias", "residual"}
    t5 = t5_op_names(1)
    assert "enc_out" in live_keys_before(t5, t5.index("dec-2nd-layernorm"))       # still needed by cross-attention
    assert "enc_out" not in live_keys_before(t5, t5.index("dec-MLP-GEMM-1"))      # last use was dec-attention-qkv-2
    rn = resnet_op_names(ResNetConfig(blocks=(1, 1, 1, 1)))
    assert set(live_keys_before(rn, rn.index("block-0-0-conv2"))) == {"x", "residual"}


def test_t5_variants_agree():
    ov = dict(hidden_dropout=0.0, attention_dropout=0.0, max_tp=1)
    runs = []
    for fuse, rc in ((True, 0), (True, 1), (False, 0)):
        t = Trainer(tiny_t5_plan(recompute=rc), model_overrides=ov, fuse=fuse, lr_warmup_steps=0, device="cpu")
        runs.append([t.loss_value(t.train_step(t5_batch(4, 64, 32, 256, seed=1))) for _ in range(3)])
    assert runs[0][-1] < runs[0][0]
    for other in runs[1:]:
        assert max(abs(a - b) for a, b in zip(runs[0], other)) < 2e-3


def test_resnet_variants_agree():
    ov = dict(image_size=64, num_classes=16)
    runs = []
    for fuse, rc in ((True, 0), (True, 1), (False, 0)):
        t = Trainer(tiny_resnet_plan(recompute=rc, global_bs=16, micro_bs=8), model_overrides=ov, fuse=fuse,
                    lr_warmup_steps=0, device="cpu", lr=1e-3)
        runs.append([t.loss_value(t.train_step(resnet_batch(16, 64, 16, seed=1))) for _ in range(3)])
    assert runs[0][-1] < runs[0][0]
    assert max(abs(a - b) for a, b in zip(runs[0], runs[1])) < 1e-4      # recompute replays exactly
    assert max(abs(a - b) for a, b in zip(runs[0], runs[2])) < 3e-2      # fusion only changes rounding
