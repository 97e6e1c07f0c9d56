"""Inverse-cloze biencoder: the in-batch retrieval loss, learning to match queries with their blocks, data-parallel
ranks scoring against each other's blocks, and the trained encoder as the embedder of the evidence index."""
import math

import numpy as np
import torch

from dist_utils import run_ranks
from helpers import tiny_ict_plan

KW = dict(layers=2, seq=16, hidden=64, heads=2, head_dim=32, vocab=128, global_bs=16, micro_bs=16)
OV = dict(hidden_dropout=0.0, attention_dropout=0.0)


def _pairs(n, seed):
    """Query i and block i share a random 'topic' token pattern; everything else is noise."""
    g = torch.Generator().manual_seed(seed)
    topic = torch.randint(10, 128, (n, 6), generator=g)
    ids = torch.zeros(2 * n, 16, dtype=torch.int64)
    for i in range(n):
        for row in (2 * i, 2 * i + 1):
            noise = torch.randint(10, 128, (9,), generator=g)
            ids[row] = torch.cat([torch.tensor([2]), topic[i], noise])[:16]
    return {"ids": ids, "types": torch.zeros_like(ids), "enc_lens": torch.full((2 * n,), 16, dtype=torch.int32),
            "labels": torch.arange(n).repeat_interleave(2)}


def _trainer(plan, rank=0, world=1, lr=3e-3, **kw):
    from superscaler_b200.runtime.trainer import Trainer
    return Trainer(plan, rank=rank, world_size=world, device="cpu", model_overrides=OV, lr_warmup_steps=0, lr=lr, **kw)


def test_loss_is_the_in_batch_softmax_and_training_learns_the_pairs():
    t = _trainer(tiny_ict_plan(**KW))
    b = _pairs(8, seed=1)
    first = t.loss_value(t.train_step(b))
    assert abs(first - math.log(8)) < 0.5                     # untrained: near-uniform over the 8 blocks of the batch
    emb = t.embed(b)
    assert emb.shape == (16, 16)
    q, c = emb[0::2].float(), emb[1::2].float()
    want = float(torch.nn.functional.cross_entropy(q @ c.t(), torch.arange(8)))
    again = t.loss_value(t.train_step(b))                      # the loss of the weights embed() just saw
    assert abs(again - want) < 2e-2, (again, want)
    for _ in range(40):
        last = t.loss_value(t.train_step(b))
    assert last < 0.5 * first, (first, last)
    emb = t.embed(b).float()
    assert ((emb[0::2] @ emb[1::2].t()).argmax(1) == torch.arange(8)).float().mean() >= 0.75


def _reduced_grad(t, batch):
    t.forward_backward(t.to_device(batch))
    t._fold_autograd_grads()
    t.optimizer.reduce_gradients()
    return t.store.grad.clone()


def _dp_worker(rank, world, plan, want):
    want_grad, want_losses = want
    t = _trainer(plan, rank, world, shard_optimizer=False)      # every rank keeps the whole reduced gradient
    # the embeddings of both ranks are gathered before the scores are taken: every query sees all 8 blocks, and the
    # averaged gradient is the gradient of that one loss (same size, not half of it)
    g = _reduced_grad(t, _pairs(8, seed=1))
    assert float((g - want_grad).norm()) < 2e-2 * float(want_grad.norm()), (rank, float(g.norm()), float(want_grad.norm()))
    t.store.zero_grad()
    got = [t.loss_value(t.train_step(_pairs(8, seed=1))) for _ in range(3)]
    assert all(abs(a - b) < 3e-2 for a, b in zip(got, want_losses)), (rank, got, want_losses)


def test_data_parallel_ranks_score_against_the_blocks_of_all_ranks():
    t = _trainer(tiny_ict_plan(**KW))
    grad = _reduced_grad(t, _pairs(8, seed=1))
    t.store.zero_grad()
    losses = [t.loss_value(t.train_step(_pairs(8, seed=1))) for _ in range(3)]
    assert abs(losses[0] - math.log(8)) < 0.5 and losses[2] < losses[0]
    run_ranks(_dp_worker, 2, tiny_ict_plan(**KW, num_gpus=(2,), tp=[1]), (grad, losses))


def test_trained_encoder_is_the_embedder_of_the_evidence_index(tmp_path):
    from superscaler_b200.data import retrieval as R
    t = _trainer(tiny_ict_plan(**KW))
    b = _pairs(8, seed=3)
    for _ in range(30):
        t.train_step(b)
    blocks_ids = b["ids"][1::2]

    def embed(ids, mask):
        return t.embed({"ids": ids, "types": torch.zeros_like(ids), "enc_lens": mask.sum(1).to(torch.int32)})

    store = R.EmbeddingStore(str(tmp_path), 0)
    store.add(torch.arange(100, 108), embed(blocks_ids, torch.ones_like(blocks_ids, dtype=torch.bool)))
    store.save_shard()
    store.merge_shards_and_save(1)
    ids, emb = R.EmbeddingStore.load(str(tmp_path))
    index = R.MIPSIndex(ids, emb)
    q = embed(b["ids"][0::2], torch.ones(8, 16, dtype=torch.bool))
    _, found = index.search(q, 1)
    assert (found[:, 0] == torch.arange(100, 108)).float().mean() >= 0.75


def test_pairs_from_a_text_corpus_and_a_titles_corpus(tmp_path):
    """`make_ict_batch_fn`: text and titles preprocessed into two sentence corpora; every block opens with
    [CLS] title [SEP], the query is a sentence of the same document, and a training step runs on the batch."""
    import json
    from superscaler_b200.data.preprocess import main as preprocess_main
    from superscaler_b200.data.sentences import SpecialTokens
    from superscaler_b200.runtime.pretrain import make_ict_batch_fn
    words = ["[PAD]", "[UNK]", "[CLS]", "[SEP]", "[MASK]", "."] + [f"w{i}" for i in range(40)] + [f"t{i}" for i in range(12)]
    (tmp_path / "vocab.txt").write_text("\n".join(words) + "\n")
    rng = np.random.RandomState(0)
    rows = []
    for d in range(12):
        sents = [" ".join(f"w{int(x)}" for x in rng.randint(0, 40, size=4)) + " ." for _ in range(4)]
        rows.append({"text": " ".join(sents), "title": f"t{d}"})
    (tmp_path / "in.jsonl").write_text("\n".join(json.dumps(r) for r in rows))
    for key, name in (("text", "body"), ("title", "titles")):
        preprocess_main(["--input", str(tmp_path / "in.jsonl"), "--json-key", key, "--output", str(tmp_path / name),
                         "--split-sentences", "--tokenizer-type", "BertWordPieceLowerCase",
                         "--vocab-file", str(tmp_path / "vocab.txt")])
    t = _trainer(tiny_ict_plan(**{**KW, "global_bs": 8, "micro_bs": 8}))
    special = SpecialTokens(cls=2, sep=3, mask=4, pad=0)
    fn = make_ict_batch_fn(t, str(tmp_path / "body"), str(tmp_path / "titles"), train_iters=4, seed=3, special=special,
                           split="10,2,0", eval_samples=8)
    b = fn(0)
    assert b["ids"].shape == (8, 16) and b["labels"].tolist() == [0, 0, 1, 1, 2, 2, 3, 3]
    title_ids = set(range(46, 58))
    for k in range(4):
        query, block = b["ids"][2 * k].tolist(), b["ids"][2 * k + 1].tolist()
        assert query[0] == 2 and block[0] == 2 and block[1] in title_ids and block[2] == 3
        assert int(b["enc_lens"][2 * k]) == 7                    # [CLS] + 5 word pieces + [SEP]
        assert 46 + 10 > block[1]                                 # training part: documents 0-9 only
    held = fn.valid(0)
    assert all(row[1] in (56, 57) for row in held["ids"][1::2].tolist())      # validation part: documents 10, 11
    assert fn.test is None
    assert math.isfinite(t.loss_value(t.train_step(b)))


def test_inverse_cloze_command_line_with_titles_and_a_held_out_part(tmp_path, capsys):
    import json
    import re
    from superscaler_b200.data.preprocess import main as preprocess_main
    from superscaler_b200.runtime import pretrain
    words = ["[PAD]", "[UNK]", "[CLS]", "[SEP]", "[MASK]", "."] + [f"w{i}" for i in range(40)] + [f"t{i}" for i in range(12)]
    (tmp_path / "vocab.txt").write_text("\n".join(words) + "\n")
    rng = np.random.RandomState(0)
    rows = [{"text": " ".join(" ".join(f"w{int(x)}" for x in rng.randint(0, 40, size=4)) + " ." for _ in range(4)),
             "title": f"t{d}"} for d in range(12)]
    (tmp_path / "in.jsonl").write_text("\n".join(json.dumps(r) for r in rows))
    for key, name in (("text", "body"), ("title", "titles")):
        preprocess_main(["--input", str(tmp_path / "in.jsonl"), "--json-key", key, "--output", str(tmp_path / name),
                         "--split-sentences", "--output-format", "megatron", "--tokenizer-type", "BertWordPieceLowerCase",
                         "--vocab-file", str(tmp_path / "vocab.txt")])
    plan = tmp_path / "ict_tiny_1stages.json"
    plan.write_text(json.dumps(tiny_ict_plan(**{**KW, "global_bs": 8, "micro_bs": 8})))
    pretrain.main(["--flexpipe-config", str(plan), "--train-iters", "4", "--data-path", str(tmp_path / "body"),
                   "--titles-data-path", str(tmp_path / "titles"), "--vocab-file", str(tmp_path / "vocab.txt"),
                   "--split", "10,2,0", "--eval-interval", "2", "--eval-iters", "1", "--query-in-block-prob", "0.5",
                   "--hidden-dropout", "0", "--attention-dropout", "0", "--num-workers", "2"])
    out = capsys.readouterr().out
    assert len(re.findall(r"lm loss: ([0-9.E+-]+)", out)) == 4
    assert len(re.findall(r"validation loss at iteration", out)) == 2
