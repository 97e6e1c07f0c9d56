"""Sampling filters and the generation loop on a tiny GPT (reference: runtime/megatron/text_generation_utils.py)."""
import torch

from superscaler_b200.data.synthetic import gpt_batch
from superscaler_b200.runtime.generation import filter_logits, generate, sample_next
from superscaler_b200.runtime.trainer import Trainer

from helpers import tiny_gpt_plan


def test_top_k_and_top_p_filters():
    logits = torch.log(torch.tensor([[0.5, 0.25, 0.15, 0.07, 0.03]]))
    k2 = filter_logits(logits, top_k=2)
    assert torch.isfinite(k2[0]).tolist() == [True, True, False, False, False]
    p = filter_logits(logits, top_p=0.8)           # 0.5 + 0.25 < 0.8 <= 0.5 + 0.25 + 0.15
    assert torch.isfinite(p[0]).tolist() == [True, True, True, False, False]
    tiny = filter_logits(logits, top_p=1e-6)
    assert torch.isfinite(tiny[0]).tolist() == [True, False, False, False, False]
    shuffled = logits[:, [3, 0, 4, 2, 1]]
    assert torch.isfinite(filter_logits(shuffled, top_p=0.8)[0]).tolist() == [False, True, False, True, True]
    assert sample_next(logits, greedy=True).tolist() == [0]
    g = torch.Generator().manual_seed(0)
    draws = [int(sample_next(logits, top_k=2, generator=g)) for _ in range(200)]
    assert set(draws) == {0, 1} and draws.count(0) > draws.count(1)


def test_generation_on_a_tiny_gpt_learns_a_repeating_pattern():
    kw = dict(layers=2, seq=32, hidden=64, heads=2, head_dim=32, vocab=64, global_bs=8, micro_bs=8)
    t = Trainer(tiny_gpt_plan(**kw), model_overrides=dict(hidden_dropout=0.0, attention_dropout=0.0),
                lr_warmup_steps=0, device="cpu", lr=3e-3, lr_style="constant")
    # the corpus is the periodic sequence 5, 6, ..., 12, 5, 6, ...; the model learns next = f(previous)
    period = torch.arange(5, 13)
    rows = torch.stack([period.roll(-i).repeat(5)[:33] for i in range(8)])
    batch = {"ids": rows[:, :-1].contiguous(), "labels": rows[:, 1:].contiguous()}
    first = t.loss_value(t.train_step(batch))
    for _ in range(60):
        last = t.loss_value(t.train_step(batch))
    assert last < 0.2 * first
    ev = t.evaluate([batch])
    assert abs(ev["lm loss"] - last) < 0.5 and ev["lm loss ppl"] >= 1.0
    lg = t.logits(batch["ids"])
    assert lg.shape[:2] == (8, 32) and lg.shape[2] >= 64
    out = generate(t, [[5, 6, 7], [9, 10]], max_new_tokens=6, greedy=True, vocab_size=64)
    assert out[0] == [5, 6, 7, 8, 9, 10, 11, 12, 5] and out[1] == [9, 10, 11, 12, 5, 6, 7, 8]
    stop = generate(t, [[5, 6, 7]], max_new_tokens=6, greedy=True, eod=9, vocab_size=64)
    assert stop[0] == [5, 6, 7, 8, 9]
    # sampling with a tiny nucleus equals greedy decoding
    same = generate(t, [[5, 6, 7]], max_new_tokens=4, top_p=1e-4, vocab_size=64)
    assert same[0] == out[0][:7]


def _tp_logits_worker(rank, world, plan, want):
    t = Trainer(plan, rank=rank, world_size=world, model_overrides=dict(hidden_dropout=0.0, attention_dropout=0.0,
                                                                        max_tp=2), device="cpu")
    ids = gpt_batch(4, 32, 64, seed=3)["ids"]
    got = t.logits(ids)
    assert got.shape == want.shape and float((got.float() - want.float()).abs().max()) < 2e-2
    out = generate(t, [[5, 6, 7]], max_new_tokens=3, greedy=True, vocab_size=64)
    assert len(out[0]) == 6


def test_logits_and_generation_under_tensor_parallelism():
    """The vocabulary-parallel LM head gathers its logit shards: two ranks give the single-process logits."""
    import sys, os
    sys.path.insert(0, os.path.dirname(__file__))
    from dist_utils import run_ranks
    kw = dict(layers=2, seq=32, hidden=64, heads=2, head_dim=32, vocab=64, global_bs=4, micro_bs=4)
    single = Trainer(tiny_gpt_plan(**kw), model_overrides=dict(hidden_dropout=0.0, attention_dropout=0.0, max_tp=2),
                     device="cpu")
    want = single.logits(gpt_batch(4, 32, 64, seed=3)["ids"])
    run_ranks(_tp_logits_worker, 2, tiny_gpt_plan(**kw, num_gpus=(2,), tp=[2]), want)


def _plans_logits_worker(rank, world, plans, want, want_gen):
    for plan in plans:
        t = Trainer(plan, rank=rank, world_size=world, model_overrides=dict(hidden_dropout=0.0, attention_dropout=0.0,
                                                                            max_tp=2), device="cpu")
        got = t.logits(gpt_batch(4, 32, 64, seed=3)["ids"])
        assert got.shape == want.shape and float((got.float() - want.float()).abs().max()) < 2e-2, (rank, plan)
        # one prompt: fewer rows than data-parallel ranks, padded inside logits()
        assert generate(t, [[5, 6, 7]], max_new_tokens=3, greedy=True, vocab_size=64) == want_gen, (rank, plan)


def test_logits_and_generation_under_pipeline_and_data_parallel_plans():
    """Every rank of a pipeline / data-parallel / mixed-layout plan gets the single-process logits and continues a
    prompt with the same tokens."""
    import sys, os
    sys.path.insert(0, os.path.dirname(__file__))
    from dist_utils import run_ranks
    kw = dict(layers=2, seq=32, hidden=64, heads=2, head_dim=32, vocab=64, global_bs=4, micro_bs=4)
    single = Trainer(tiny_gpt_plan(**kw), model_overrides=dict(hidden_dropout=0.0, attention_dropout=0.0, max_tp=2),
                     device="cpu")
    want = single.logits(gpt_batch(4, 32, 64, seed=3)["ids"])
    want_gen = generate(single, [[5, 6, 7]], max_new_tokens=3, greedy=True, vocab_size=64)
    mixed = tiny_gpt_plan(**kw, num_gpus=(2,), tp=[2])
    n = mixed["num_ops_in_each_stage"][0]
    tp = [1] * 12 + [2] * (n - 12)          # data parallel first, tensor parallel (and a sharded LM head) after
    mixed.update(model_parallel_size_of_each_op=[tp], data_parallel_size_of_each_op=[[2 // t for t in tp]],
                 resharding_stages=[True])
    run_ranks(_plans_logits_worker, 2, [tiny_gpt_plan(**kw, num_gpus=(2,), tp=[1]), tiny_gpt_plan(**kw, num_gpus=(1, 1)),
                                        mixed], want, want_gen)
    run_ranks(_plans_logits_worker, 4, [tiny_gpt_plan(**kw, num_gpus=(2, 2), tp=[1, 2]),
                                        tiny_gpt_plan(**kw, num_gpus=(1, 2, 1), tp=[1, 1, 1])], want, want_gen)


def test_generation_command_line(tmp_path, capsys):
    """Prompts from flags and from a file, then unconditional samples, through the tiny byte-level BPE vocabulary."""
    import json
    import sys, os
    sys.path.insert(0, os.path.dirname(__file__))
    from test_tokenizer_cpu import _bpe_files
    from superscaler_b200.runtime import generation
    vf, mf, vocab, _ = _bpe_files(tmp_path)
    plan = tmp_path / "plan.json"
    plan.write_text(json.dumps(tiny_gpt_plan(layers=1, seq=32, hidden=64, heads=2, head_dim=32, vocab=384,
                                             global_bs=2, micro_bs=2)))
    (tmp_path / "prompts.txt").write_text("newer\n\nlow low\n")
    out = tmp_path / "out.json"
    generation.main(["--flexpipe-config", str(plan), "--vocab-file", vf, "--merge-file", mf, "--prompt", "lower new",
                     "--sample-input-file", str(tmp_path / "prompts.txt"), "--sample-output-file", str(out),
                     "--out-seq-length", "4", "--top_k", "5", "--temperature", "0.8"])
    texts = json.loads(out.read_text())
    assert len(texts) == 3 and texts[0].startswith("lower new") and texts[1].startswith("newer")
    assert texts[2].startswith("low low") and "--- sample 2 ---" in capsys.readouterr().out
    generation.main(["--flexpipe-config", str(plan), "--vocab-file", vf, "--merge-file", mf, "--num-samples", "2",
                     "--out-seq-length", "3", "--greedy", "--sample-output-file", str(out)])
    texts = json.loads(out.read_text())
    assert len(texts) == 2 and texts[0] == texts[1]
