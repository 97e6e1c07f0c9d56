"""Vision transformer as an op-list model: patch order, the loss against plain PyTorch, training, and data / tensor /
pipeline parallel plans against one process (gloo)."""
import math

import torch

from dist_utils import run_ranks
from helpers import tiny_vit_plan

KW = dict(layers=2, hidden=64, heads=2, head_dim=32, global_bs=8, micro_bs=4)
OV = dict(hidden_dropout=0.0, attention_dropout=0.0)


def _batch(seed=1):
    from superscaler_b200.data.synthetic import resnet_batch
    return resnet_batch(KW["global_bs"], 32, 10, seed=seed)


def test_loss_matches_a_plain_pytorch_vit():
    from superscaler_b200.ops import functional as F
    from superscaler_b200.runtime.trainer import Trainer
    t = Trainer(tiny_vit_plan(**dict(KW, micro_bs=8)), device="cpu", model_overrides=OV, lr_warmup_steps=0)
    assert t.cfg.seq_length == 17
    b = _batch(2)
    st = t.microbatch_inputs(t.to_device(b), 0)
    t.stage.forward(st)
    got = float(st["loss"].detach())
    byop = {}
    for k, v in t.store.params.items():
        _, idx, key = k.split(".", 2)
        byop.setdefault(int(idx), {})[key] = v.detach().float()
    img = b["images"].float()
    B, H, NH, HD, S = img.shape[0], KW["hidden"], KW["heads"], KW["head_dim"], 17
    e = byop[0]
    # patch (r, c) of an image, flattened (row, column, channel): unfold with channels last
    patches = img.unfold(1, 8, 8).unfold(2, 8, 8)                       # [B, 4, 4, 3, 8, 8]
    patches = patches.permute(0, 1, 2, 4, 5, 3).reshape(B, 16, 8 * 8 * 3)
    x = patches @ e["linear_encoder.weight"].t() + e["linear_encoder.bias"]
    x = torch.cat([e["cls_token"].expand(B, 1, H), x], 1) + e["position_embeddings.weight"][None]
    x = x.reshape(B * S, H)
    ln = lambda v, p: torch.nn.functional.layer_norm(v, (H,), p["layernorm.weight"], p["layernorm.bias"], 1e-5)
    for layer in range(KW["layers"]):
        o = 1 + 13 * layer
        h = ln(x, byop[o])
        qkv = h @ byop[o + 1]["query_key_value.weight"].reshape(-1, H).t() + byop[o + 1]["query_key_value.bias"].reshape(-1)
        w = NH * HD
        q, k, v = (qkv[:, i * w:(i + 1) * w].view(B, S, NH, HD).permute(0, 2, 1, 3) for i in range(3))
        p = torch.softmax((q @ k.transpose(-1, -2)) / math.sqrt(HD), -1)
        x = x + (p @ v).permute(0, 2, 1, 3).reshape(B * S, w) @ byop[o + 6]["dense.weight"].t() + byop[o + 6]["dense.bias"]
        h = ln(x, byop[o + 8])
        u = F._gelu_tanh(h @ byop[o + 9]["dense_h_to_4h.weight"].t() + byop[o + 9]["dense_h_to_4h.bias"])
        x = x + u @ byop[o + 11]["dense_4h_to_h.weight"].t() + byop[o + 11]["dense_4h_to_h.bias"]
    last = 1 + 13 * KW["layers"]
    x = ln(x, byop[last])
    hp = byop[last + 1]
    cls = torch.tanh(x.view(B, S, H)[:, 0] @ hp["head.dense_in.weight"].t() + hp["head.dense_in.bias"])
    want = float(torch.nn.functional.cross_entropy(cls @ hp["head.dense_out.weight"].t() + hp["head.dense_out.bias"],
                                                   b["labels"]))
    assert abs(got - want) < 2e-2 * max(1.0, abs(want)), (got, want)


def _losses(plan, rank=0, world=1, steps=3):
    from superscaler_b200.runtime.trainer import Trainer
    t = Trainer(plan, rank=rank, world_size=world, device="cpu", model_overrides=OV, lr_warmup_steps=0, lr=2e-3)
    return [t.loss_value(t.train_step(_batch(1))) for _ in range(steps)]


def test_vit_trains():
    ls = _losses(tiny_vit_plan(**KW), steps=6)
    assert all(math.isfinite(v) for v in ls) and ls[-1] < ls[0]


def _worker(rank, world, plans, want):
    for name, plan in plans.items():
        got = _losses(plan, rank, world)
        assert max(abs(a - b) for a, b in zip(got, want)) < 6e-3, (rank, name, got, want)


def test_data_tensor_and_pipeline_parallel_plans_match_one_process():
    want = _losses(tiny_vit_plan(**KW))
    plans = {"dp": tiny_vit_plan(**KW, num_gpus=(2,), tp=[1]),
             "tp": tiny_vit_plan(**KW, num_gpus=(2,), tp=[2]),
             "pp": tiny_vit_plan(**KW, num_gpus=(1, 1))}
    run_ranks(_worker, 2, plans, want, timeout=600)


def _accuracy(plan, rank=0, world=1):
    """Evaluation of the untrained and of the trained model on the training batch: loss and top-1 accuracy."""
    from superscaler_b200.runtime.trainer import Trainer
    t = Trainer(plan, rank=rank, world_size=world, device="cpu", model_overrides=OV, lr_warmup_steps=0, lr=2e-3)
    before = t.evaluate([_batch(1)])
    for _ in range(25):
        t.train_step(_batch(1))
    return before, t.evaluate([_batch(1)])


def _accuracy_worker(rank, world, plans, want):
    for name, plan in plans.items():
        before, after = _accuracy(plan, rank, world)
        for got, ref in ((before, want[0]), (after, want[1])):
            assert set(got) == {"lm loss", "accuracy"}
            close = abs(got["lm loss"] - ref["lm loss"]) < 3e-2 and abs(got["accuracy"] - ref["accuracy"]) <= 0.26
            assert close, (rank, name, got, ref)


def test_evaluation_reports_top1_accuracy_on_every_rank_of_any_plan():
    before, after = _accuracy(tiny_vit_plan(**KW))
    b = _batch(1)
    assert 0.0 <= before["accuracy"] <= 0.5 and after["accuracy"] >= 0.75 and after["lm loss"] < before["lm loss"]
    assert abs(after["accuracy"] * b["labels"].numel() - round(after["accuracy"] * b["labels"].numel())) < 1e-4
    plans = {"dp": tiny_vit_plan(**KW, num_gpus=(2,), tp=[1]), "pp": tiny_vit_plan(**KW, num_gpus=(1, 1))}
    run_ranks(_accuracy_worker, 2, plans, (before, after), timeout=600)
