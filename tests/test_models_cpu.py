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


def test_resnet_evaluation_uses_running_statistics_and_leaves_them_alone():
    """Trainer.evaluate normalises with the running mean / variance like torch.nn.BatchNorm2d.eval() and does not
    update them (the buffers are part of a checkpoint)."""
    from superscaler_b200.models.resnet import BNOp
    from superscaler_b200.ops import conv as C
    ov = dict(image_size=64, num_classes=16)
    t = Trainer(tiny_resnet_plan(global_bs=8, micro_bs=4), model_overrides=ov, lr_warmup_steps=0, device="cpu", lr=1e-3)
    for i in range(2):
        t.train_step(resnet_batch(8, 64, 16, seed=i))
    def bn_ops():
        for op in t.stage.ops:
            for cand in (op, getattr(op, "bn_op", None), *getattr(op, "ops", ())):
                if isinstance(cand, BNOp) and cand.run_mean is not None:
                    yield cand
    before = [(o.run_mean.clone(), o.run_var.clone()) for o in bn_ops()]
    assert before, "no BatchNorm buffers found"
    a = t.evaluate([resnet_batch(8, 64, 16, seed=5)])
    b = t.evaluate([resnet_batch(8, 64, 16, seed=5)])
    after = [(o.run_mean, o.run_var) for o in bn_ops()]
    assert all(torch.equal(x[0], y[0]) and torch.equal(x[1], y[1]) for x, y in zip(before, after))
    assert a == b

    # the op against torch's module in eval mode
    torch.manual_seed(0)
    x = torch.randn(2, 5, 5, 8)
    bn = torch.nn.BatchNorm2d(8).eval()
    with torch.no_grad():
        bn.weight.uniform_(0.5, 1.5); bn.bias.uniform_(-1, 1)
        bn.running_mean.uniform_(-1, 1); bn.running_var.uniform_(0.5, 2.0)
        want = torch.relu(bn(x.permute(0, 3, 1, 2))).permute(0, 2, 3, 1)
    got = C.batch_norm_inference(x, bn.weight.detach(), bn.bias.detach(), bn.running_mean, bn.running_var,
                                 eps=bn.eps, relu=True)
    assert torch.allclose(got, want, atol=1e-5)
