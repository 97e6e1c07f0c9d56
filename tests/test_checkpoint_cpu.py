"""Checkpoint layout and resume (CPU)."""
import os

import torch

from superscaler_b200.data.synthetic import gpt_batch
from superscaler_b200.runtime import checkpointing as ck
from superscaler_b200.runtime.trainer import Trainer

from helpers import tiny_gpt_plan

NODROP = dict(hidden_dropout=0.0, attention_dropout=0.0, max_tp=1)


def _trainer():
    return Trainer(tiny_gpt_plan(), model_overrides=NODROP, lr_warmup_steps=0, device="cpu")


def _step(t, seed):
    return t.loss_value(t.train_step(gpt_batch(4, 128, 512, seed=seed)))


def test_save_layout_and_exact_resume(tmp_path):
    a = _trainer()
    for i in range(2):
        _step(a, i)
    path = ck.save_checkpoint(a, str(tmp_path))
    assert path.endswith(os.path.join("iter_0000002", "mp_rank_00", "model_optim_rng.pt"))
    assert ck.read_tracker(str(tmp_path)) == 2
    sd = torch.load(path, weights_only=False)
    assert sd["checkpoint_version"] == 3.0 and sd["iteration"] == 2 and "plan" in sd
    assert all(k.startswith("language_model.ops.") for k in sd["model"])
    assert "language_model.ops.0.word_embeddings.weight" in sd["model"]
    cont = [_step(a, 10 + i) for i in range(2)]
    b = _trainer()
    assert ck.load_checkpoint(b, str(tmp_path)) == 2
    resumed = [_step(b, 10 + i) for i in range(2)]
    assert cont == resumed


def test_reassemble_under_plan(tmp_path):
    a = _trainer()
    _step(a, 0)
    ck.save_checkpoint(a, str(tmp_path))
    full = ck.merge_tp_shards(str(tmp_path), 1)
    assert full["0.word_embeddings.weight"].shape == (512, 128)
    b = _trainer()
    ck.load_under_plan(b, str(tmp_path))
    assert torch.equal(a.store.master, b.store.master)
