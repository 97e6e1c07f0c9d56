"""Checkpoint layout and resume (CPU)."""
import os

import pytest
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


def test_export_to_upstream_megatron_names_and_back(tmp_path):
    """A checkpoint merged from its shards converts to the upstream GPT parameter names (QKV rows interleaved per
    head) and back without loss; the converted QKV projects like the original."""
    import torch
    from superscaler_b200.runtime import checkpointing
    from superscaler_b200.runtime.megatron_names import export_megatron_gpt, import_megatron_gpt
    from superscaler_b200.runtime.trainer import Trainer
    from helpers import tiny_gpt_plan
    t = Trainer(tiny_gpt_plan(layers=2), device="cpu")
    checkpointing.save_checkpoint(t, str(tmp_path))
    full = checkpointing.merge_tp_shards(str(tmp_path), 0)
    heads = t.cfg.heads
    up = export_megatron_gpt(full, t.op_names, heads)
    assert "language_model.embedding.word_embeddings.weight" in up
    assert "language_model.encoder.layers.1.self_attention.query_key_value.weight" in up
    assert "language_model.encoder.layers.0.mlp.dense_4h_to_h.bias" in up
    assert "language_model.encoder.final_layernorm.weight" in up
    assert len(up) == 2 + 12 * 2 + 2
    legacy = export_megatron_gpt(full, t.op_names, heads, legacy=True)
    assert "language_model.transformer.layers.0.attention.dense.weight" in legacy
    back = import_megatron_gpt(up, t.op_names, heads)
    assert all(torch.equal(back[k], full[k]) for k in back) and set(back) == {k for k in full if k in back}
    # per-head interleaving: head 1's K rows of ours are rows [1 * 3 * hd + hd, ... + 2 * hd) upstream
    ours = next(v for k, v in full.items() if k.endswith("query_key_value.weight"))
    theirs = up["language_model.encoder.layers.0.self_attention.query_key_value.weight"]
    hd = ours.shape[1] // heads
    assert torch.equal(theirs[1 * 3 * hd + hd: 1 * 3 * hd + 2 * hd], ours[1, hd:2 * hd])
    x = torch.randn(5, ours.shape[2])
    q_ours = (x @ ours[0].float().t()).view(5, heads, hd)
    q_theirs = (x @ theirs.float().t()).view(5, heads, 3, hd)[:, :, 0]
    assert torch.allclose(q_ours, q_theirs)


def test_gpt_logits_match_huggingface_gpt2(tmp_path):
    """An independent implementation as oracle: the exported weights loaded into transformers' GPT2LMHeadModel
    give the same logits as this framework's op-list GPT (up to the bf16 rounding its CPU path emulates)."""
    import pytest
    import torch
    transformers = pytest.importorskip("transformers")
    from superscaler_b200.data.synthetic import gpt_batch
    from superscaler_b200.runtime import checkpointing
    from superscaler_b200.runtime.hf_export import hf_gpt2_config, to_hf_gpt2
    from superscaler_b200.runtime.trainer import Trainer
    from helpers import tiny_gpt_plan
    plan = tiny_gpt_plan(layers=2, seq=64, hidden=128, heads=2, head_dim=64, vocab=512, global_bs=4, micro_bs=4)
    t = Trainer(plan, device="cpu", model_overrides=dict(hidden_dropout=0.0, attention_dropout=0.0),
                lr_warmup_steps=0, lr=1e-3)
    batch = gpt_batch(4, 64, 512, seed=3)
    for _ in range(2):                       # a trained model: biases and LayerNorm parameters are no longer trivial
        t.train_step(batch)
    checkpointing.save_checkpoint(t, str(tmp_path))
    full = checkpointing.merge_tp_shards(str(tmp_path), t.iteration)
    hf = transformers.GPT2LMHeadModel(hf_gpt2_config(t.cfg)).eval()
    missing, unexpected = hf.load_state_dict(to_hf_gpt2(full, t.op_names), strict=False)
    assert not unexpected and all(k.endswith(("attn.bias", "attn.masked_bias")) for k in missing)
    with torch.no_grad():
        want = hf(batch["ids"]).logits.float()
    got = t.logits(batch["ids"]).float()
    rel = float((got - want).norm() / want.norm())
    assert rel < 2e-2, rel
    agree = float((got.argmax(-1) == want.argmax(-1)).float().mean())
    assert agree > 0.9, agree


def _save_worker(rank, world, plan, root):
    from superscaler_b200.data.synthetic import gpt_batch
    from superscaler_b200.runtime.trainer import Trainer
    t = Trainer(plan, rank=rank, world_size=world, device="cpu", lr_warmup_steps=0, lr=1e-3,
                model_overrides=dict(hidden_dropout=0.0, attention_dropout=0.0, max_tp=2))
    for i in range(2):
        t.train_step(gpt_batch(4, 128, 512, seed=i))
    ck.save_checkpoint(t, root)


@pytest.mark.parametrize("name,kw,world", [("pp2", dict(num_gpus=(1, 1)), 2), ("tp2", dict(num_gpus=(2,), tp=[2]), 2),
                                           ("pp2_tp2", dict(num_gpus=(2, 2), tp=[2, 2]), 4)])
def test_checkpoints_of_parallel_plans_reload_on_one_rank(tmp_path, name, kw, world):
    """Shards written by pipeline / tensor parallel runs merge into the weights the single-process run has after
    the same two steps (the tied embedding copy of the last stage included)."""
    from dist_utils import run_ranks
    from superscaler_b200.data.synthetic import gpt_batch
    from superscaler_b200.runtime.trainer import Trainer
    from helpers import tiny_gpt_plan
    root = str(tmp_path / name)
    run_ranks(_save_worker, world, tiny_gpt_plan(**kw), root)
    ov = dict(hidden_dropout=0.0, attention_dropout=0.0, max_tp=2)
    ref = Trainer(tiny_gpt_plan(), device="cpu", lr_warmup_steps=0, lr=1e-3, model_overrides=ov)
    for i in range(2):
        ref.train_step(gpt_batch(4, 128, 512, seed=i))
    got = Trainer(tiny_gpt_plan(), device="cpu", lr_warmup_steps=0, lr=1e-3, model_overrides=ov, seed=77)
    assert ck.load_under_plan(got, root) == 2
    for n in ref.store.params:
        a, b = ref.store.state_dict()[n], got.store.state_dict()[n]
        # two Adam steps of 1e-3 move every weight by up to 2e-3 whatever the size of its gradient, so runs whose
        # tiny gradients differ in rounding may end 4e-3 apart; a wrongly placed shard would differ by ~0.03
        assert torch.allclose(a, b, atol=5e-3), (n, float((a - b).abs().max()))
    batch = gpt_batch(4, 128, 512, seed=9)
    la, lb = ref.loss_value(ref.train_step(batch)), got.loss_value(got.train_step(batch))
    assert abs(la - lb) < 2e-2


def _model_bits(model):
    from superscaler_b200.data import synthetic as syn
    from helpers import tiny_bert_plan, tiny_resnet_plan, tiny_t5_plan, tiny_vit_plan
    if model == "bert":
        return (lambda **kw: tiny_bert_plan(seq=32, vocab=256, **kw)), \
            dict(hidden_dropout=0.0, attention_dropout=0.0, max_tp=2), (lambda seed: syn.bert_batch(4, 32, 256, seed=seed))
    if model == "vit":
        return tiny_vit_plan, dict(hidden_dropout=0.0, attention_dropout=0.0), \
            (lambda seed: syn.resnet_batch(4, 32, 10, seed=seed))
    if model == "gpt":
        return tiny_gpt_plan, dict(hidden_dropout=0.0, attention_dropout=0.0, max_tp=2), \
            (lambda seed: syn.gpt_batch(4, 128, 512, seed=seed))
    if model == "t5":
        return tiny_t5_plan, dict(hidden_dropout=0.0, attention_dropout=0.0, max_tp=2), \
            (lambda seed: syn.t5_batch(4, 64, 32, 256, seed=seed))
    return tiny_resnet_plan, dict(image_size=32, num_classes=16), \
        (lambda seed: syn.resnet_batch(4, 32, 16, seed=seed, dtype=torch.float32))


def _load_worker(rank, world, model, kw, root, want):
    plan_fn, ov, batch_fn = _model_bits(model)
    t = Trainer(plan_fn(**kw), rank=rank, world_size=world, device="cpu", lr_warmup_steps=0, lr=1e-3,
                model_overrides=ov, seed=55)
    assert ck.load_under_plan(t, root) == 2
    got = t.loss_value(t.train_step(batch_fn(9)))
    assert abs(got - want) < 2e-2 * max(1.0, abs(want)), (rank, got, want)


@pytest.mark.parametrize("model,kw,world", [("gpt", dict(num_gpus=(2,), tp=[2]), 2), ("gpt", dict(num_gpus=(1, 1)), 2),
                                            ("t5", dict(num_gpus=(2,), tp=[2]), 2), ("t5", dict(num_gpus=(1, 1)), 2),
                                            ("resnet", dict(num_gpus=(2,), tp=[2]), 2),
                                            ("resnet", dict(num_gpus=(1, 1)), 2),
                                            ("bert", dict(num_gpus=(2,), tp=[2]), 2), ("bert", dict(num_gpus=(1, 1)), 2),
                                            ("vit", dict(num_gpus=(2,), tp=[2]), 2), ("vit", dict(num_gpus=(1, 1)), 2)])
def test_one_rank_checkpoint_loads_under_parallel_plans(tmp_path, model, kw, world):
    """The other direction: a checkpoint written by one rank is re-sliced for tensor / pipeline parallel plans of
    every model family; the next step's loss equals the single-process continuation."""
    from dist_utils import run_ranks
    plan_fn, ov, batch_fn = _model_bits(model)
    root = str(tmp_path / "ckpt")
    ref = Trainer(plan_fn(), device="cpu", lr_warmup_steps=0, lr=1e-3, model_overrides=ov)
    for i in range(2):
        ref.train_step(batch_fn(i))
    ck.save_checkpoint(ref, root)
    want = ref.loss_value(ref.train_step(batch_fn(9)))
    run_ranks(_load_worker, world, model, kw, root, want)


def _mixed_plan(first_tp):
    plan = tiny_gpt_plan(num_gpus=(2,), tp=[2])
    n = plan["num_ops_in_each_stage"][0]
    tp = [first_tp] * 10 + [3 - first_tp] * (n - 10)
    plan["model_parallel_size_of_each_op"] = [tp]
    plan["data_parallel_size_of_each_op"] = [[2 // t for t in tp]]
    plan["resharding_stages"] = [True]
    return plan


def _resume_worker(rank, world, plan, root):
    ov = dict(hidden_dropout=0.0, attention_dropout=0.0, max_tp=2)
    a = Trainer(plan, rank=rank, world_size=world, device="cpu", lr_warmup_steps=0, lr=1e-3, model_overrides=ov)
    for i in range(2):
        a.train_step(gpt_batch(4, 128, 512, seed=i))
    ck.save_checkpoint(a, root)
    b = Trainer(plan, rank=rank, world_size=world, device="cpu", lr_warmup_steps=0, lr=1e-3, model_overrides=ov, seed=9)
    assert ck.load_checkpoint(b, root) == 2
    assert torch.equal(a.store.master, b.store.master)
    la = a.loss_value(a.train_step(gpt_batch(4, 128, 512, seed=5)))
    lb = b.loss_value(b.train_step(gpt_batch(4, 128, 512, seed=5)))
    assert abs(la - lb) < 1e-6


@pytest.mark.parametrize("first_tp", [1, 2])
def test_checkpoint_of_a_stage_that_mixes_tensor_parallel_degrees(tmp_path, first_tp):
    """Ops 0..9 on (tp, dp) = (1, 2) and the rest on (2, 1), or the other way round: every rank holds the only copy
    of some shard, so every rank writes; the same plan resumes exactly and one rank reloads the merged weights."""
    from dist_utils import run_ranks
    root = str(tmp_path / "ckpt")
    run_ranks(_resume_worker, 2, _mixed_plan(first_tp), root)
    ov = dict(hidden_dropout=0.0, attention_dropout=0.0, max_tp=2)
    ref = Trainer(tiny_gpt_plan(), device="cpu", lr_warmup_steps=0, lr=1e-3, model_overrides=ov)
    for i in range(2):
        ref.train_step(gpt_batch(4, 128, 512, seed=i))
    got = Trainer(tiny_gpt_plan(), device="cpu", lr_warmup_steps=0, lr=1e-3, model_overrides=ov, seed=77)
    assert ck.load_under_plan(got, root) == 2
    batch = gpt_batch(4, 128, 512, seed=9)
    assert abs(ref.loss_value(ref.train_step(batch)) - got.loss_value(got.train_step(batch))) < 2e-2


def test_batchnorm_running_statistics_travel_with_the_checkpoint(tmp_path):
    from superscaler_b200.data.synthetic import resnet_batch
    from helpers import tiny_resnet_plan
    ov = dict(image_size=64, num_classes=16)
    a = Trainer(tiny_resnet_plan(global_bs=8, micro_bs=4), device="cpu", lr_warmup_steps=0, model_overrides=ov)
    for i in range(2):
        a.train_step(resnet_batch(8, 64, 16, seed=i, dtype=torch.float32))
    ck.save_checkpoint(a, str(tmp_path))
    b = Trainer(tiny_resnet_plan(global_bs=8, micro_bs=4), device="cpu", lr_warmup_steps=0, model_overrides=ov, seed=3)
    assert ck.load_checkpoint(b, str(tmp_path)) == 2
    stats_a, stats_b = ck._buffers(a), ck._buffers(b)
    assert len(stats_a) >= 2 * 13 and stats_a.keys() == stats_b.keys()       # 12 block BNs + stem (+ downsample BNs)
    assert any("downsample.bn.running_mean" in k for k in stats_a)
    for k in stats_a:
        assert torch.equal(stats_a[k], stats_b[k]), k
    assert any(float(v.abs().sum()) > 0 for k, v in stats_a.items() if k.endswith("running_mean"))
