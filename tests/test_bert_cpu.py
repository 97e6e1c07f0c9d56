"""BERT as an op-list model: the loss against a plain PyTorch restatement, training, and data / tensor / pipeline
parallel plans against the single-process run (gloo)."""
import math

import pytest
import torch

from dist_utils import run_ranks
from helpers import tiny_bert_plan

KW = dict(layers=2, seq=32, hidden=64, heads=2, head_dim=32, vocab=256, global_bs=8, micro_bs=4)
OV = dict(hidden_dropout=0.0, attention_dropout=0.0)


def _batch(seed=1):
    from superscaler_b200.data.synthetic import bert_batch
    return bert_batch(KW["global_bs"], KW["seq"], KW["vocab"], seed=seed)


def test_batch_has_two_segments_padding_and_masked_labels():
    b = _batch()
    ids, types, lens, labels, mask = b["ids"], b["types"], b["enc_lens"], b["labels"], b["loss_mask"]
    pos = torch.arange(KW["seq"])[None, :]
    real = pos < lens[:, None]
    assert (ids[~real] == 0).all() and (types[~real] == 0).all()
    assert ((labels >= 0) == (mask > 0)).all() and (mask[~real] == 0).all() and mask.sum() > 0
    assert (ids[mask > 0] == 4).all()                          # masked positions show [MASK]
    for r in range(ids.shape[0]):                              # types: zeros then ones inside the real tokens
        t = types[r, :int(lens[r])]
        assert t[0] == 0 and (t[1:] >= t[:-1]).all() and t[-1] == 1
    assert set(b["nsp"].tolist()) <= {0, 1}


def test_loss_matches_a_plain_pytorch_bert():
    """Forward of the op-list model with its own weights against attention / MLP / head written with torch ops in
    fp32: masked-LM mean over the masked positions plus the sentence-order cross entropy."""
    from superscaler_b200.ops import functional as F
    from superscaler_b200.runtime.trainer import Trainer
    plan = tiny_bert_plan(**dict(KW, micro_bs=8))
    t = Trainer(plan, device="cpu", model_overrides=OV, lr_warmup_steps=0)
    b = _batch(3)
    st = t.microbatch_inputs(t.to_device(b), 0)
    t.stage.forward(st)
    got = float(st["loss"].detach())
    byop = {}
    for k, v in t.store.params.items():
        _, idx, key = k.split(".", 2)
        byop.setdefault(int(idx), {})[key] = v.detach().float()
    ids, types, lens = b["ids"], b["types"], b["enc_lens"]
    B, S, H, NH, HD = ids.shape[0], KW["seq"], KW["hidden"], KW["heads"], KW["head_dim"]
    e = byop[0]
    x = e["word_embeddings.weight"][ids] + e["position_embeddings.weight"][torch.arange(S)][None] + \
        e["tokentype_embeddings.weight"][types]
    x = x.reshape(B * S, H)
    key_ok = (torch.arange(S)[None, :] < lens[:, None])        # [B, S]
    ln = lambda v, p: torch.nn.functional.layer_norm(v, (H,), p["layernorm.weight"], p["layernorm.bias"], 1e-5)
    for layer in range(KW["layers"]):
        o = 1 + 13 * layer
        h = ln(x, byop[o])
        qkv = h @ byop[o + 1]["query_key_value.weight"].reshape(-1, H).t() + byop[o + 1]["query_key_value.bias"].reshape(-1)
        w = NH * HD
        q, k, v = (qkv[:, i * w:(i + 1) * w].view(B, S, NH, HD).permute(0, 2, 1, 3) for i in range(3))
        sc = (q @ k.transpose(-1, -2)) / math.sqrt(HD)
        sc = sc.masked_fill(~key_ok[:, None, None, :], float("-inf"))
        ctx = (torch.softmax(sc, -1) @ v).permute(0, 2, 1, 3).reshape(B * S, w)
        x = x + ctx @ byop[o + 6]["dense.weight"].t() + byop[o + 6]["dense.bias"]
        h = ln(x, byop[o + 8])
        u = F._gelu_tanh(h @ byop[o + 9]["dense_h_to_4h.weight"].t() + byop[o + 9]["dense_h_to_4h.bias"])
        x = x + u @ byop[o + 11]["dense_4h_to_h.weight"].t() + byop[o + 11]["dense_4h_to_h.bias"]
    last = 1 + 13 * KW["layers"]
    x = ln(x, byop[last])
    hp = byop[last + 1]
    tr = F._gelu_tanh(x @ hp["lm_head.dense.weight"].t() + hp["lm_head.dense.bias"])
    tr = torch.nn.functional.layer_norm(tr, (H,), hp["lm_head.layernorm.weight"], hp["lm_head.layernorm.bias"], 1e-5)
    logits = tr @ e["word_embeddings.weight"].t()              # tied: the shared parameter is stored once, with op 0
    mask = b["loss_mask"].reshape(-1) > 0
    lm = torch.nn.functional.cross_entropy(logits[mask], b["labels"].reshape(-1)[mask])
    pooled = torch.tanh(x.view(B, S, H)[:, 0] @ hp["pooler.dense.weight"].t() + hp["pooler.dense.bias"])
    nsp = torch.nn.functional.cross_entropy(pooled @ hp["binary_head.weight"].t() + hp["binary_head.bias"], b["nsp"])
    want = float(lm + nsp)
    assert abs(got - want) < 3e-2 * max(1.0, abs(want)), (got, want)


def _losses(plan, rank=0, world=1, steps=3):
    from superscaler_b200.runtime.trainer import Trainer
    t = Trainer(plan, rank=rank, world_size=world, device="cpu", model_overrides=OV, lr_warmup_steps=0, lr=2e-3)
    return [t.loss_value(t.train_step(_batch(1))) for _ in range(steps)]


def test_bert_trains():
    ls = _losses(tiny_bert_plan(**KW), steps=6)
    assert all(math.isfinite(v) for v in ls) and ls[-1] < ls[0]


def _worker(rank, world, plans, want):
    for name, plan in plans.items():
        got = _losses(plan, rank, world)
        assert max(abs(a - b) for a, b in zip(got, want)) < 6e-3, (rank, name, got, want)


def test_data_tensor_and_pipeline_parallel_plans_match_one_process():
    want = _losses(tiny_bert_plan(**KW))
    plans = {"dp": tiny_bert_plan(**KW, num_gpus=(2,), tp=[1]),
             "tp": tiny_bert_plan(**KW, num_gpus=(2,), tp=[2]),
             "pp": tiny_bert_plan(**KW, num_gpus=(1, 1))}
    # layouts change inside the stage: tp 2 at the start, dp 2 from the middle of the first layer into the second
    # (its attention sees half the samples and must take THEIR lengths for the padding mask), tp 2 again after
    mixed = tiny_bert_plan(**KW, num_gpus=(2,), tp=[2])
    n = mixed["num_ops_in_each_stage"][0]
    tp = [1 if 9 <= i < 20 else 2 for i in range(n)]
    mixed.update(model_parallel_size_of_each_op=[tp], data_parallel_size_of_each_op=[[2 // t for t in tp]],
                 resharding_stages=[True])
    plans["tp-dp-tp"] = mixed
    run_ranks(_worker, 2, plans, want, timeout=600)


def test_text_to_sentence_corpus_to_bert_training(tmp_path):
    """Text -> `data.preprocess --split-sentences` -> BertDataset batches -> training steps."""
    import numpy as np
    from superscaler_b200.data import preprocess
    from superscaler_b200.data.sentences import SpecialTokens
    from superscaler_b200.runtime.pretrain import make_bert_batch_fn
    from superscaler_b200.runtime.trainer import Trainer
    words = ["[PAD]", "[UNK]", "[CLS]", "[SEP]", "[MASK]"] + [f"w{i}" for i in range(60)] + [".", "!", "?"]
    vocab = tmp_path / "vocab.txt"
    vocab.write_text("\n".join(words) + "\n")
    rs = np.random.RandomState(0)
    docs = []
    for _ in range(12):
        sents = [" ".join(rs.choice(words[5:65], size=rs.randint(4, 9))) + rs.choice([".", "!", "?"]) for _ in range(rs.randint(3, 7))]
        docs.append(" ".join(sents))
    (tmp_path / "docs.txt").write_text("\n".join(docs) + "\n")
    assert preprocess.split_sentences("One two. Three four!  Five?\nSix") == ["One two.", "Three four!", "Five?", "Six"]
    prefix = str(tmp_path / "corpus")
    preprocess.main(["--input", str(tmp_path / "docs.txt"), "--output", prefix, "--split-sentences", "--tokenizer-type",
                     "BertWordPieceLowerCase", "--vocab-file", str(vocab)])
    corpus = preprocess.load_sentence_corpus(prefix)
    assert len(corpus.doc_starts) == 13 and corpus.doc_starts[-1] == len(corpus.sizes) >= 36
    plan = tiny_bert_plan(**dict(KW, vocab=128))
    t = Trainer(plan, device="cpu", model_overrides=OV, lr_warmup_steps=0, lr=2e-3)
    fn = make_bert_batch_fn(t, prefix, train_iters=4, seed=5,
                            special=SpecialTokens(cls=2, sep=3, mask=4, pad=0))
    b = fn(0)
    assert b["ids"].shape == (8, KW["seq"]) and set(b["types"].unique().tolist()) <= {0, 1}
    assert (b["ids"][:, 0] == 2).all() and ((b["labels"] >= 0) == (b["loss_mask"] > 0)).all()
    assert torch.equal(fn(0)["ids"], b["ids"])                           # batch i is a function of i
    losses = [t.loss_value(t.train_step(fn(i % 2))) for i in range(4)]
    assert all(math.isfinite(v) for v in losses)
    # --mask-prob reaches the dataset: more positions to predict
    more = make_bert_batch_fn(t, prefix, train_iters=4, seed=5, special=SpecialTokens(cls=2, sep=3, mask=4, pad=0),
                              data_kw=dict(mask_prob=0.4))
    assert float(more(0)["loss_mask"].sum()) > 1.5 * float(b["loss_mask"].sum())


def test_separate_attention_ops_mask_the_padding_like_the_one_kernel_form():
    """A plan that keeps score / softmax / dropout / context as four ops (here: fusion switched off) must give padded
    keys no weight either: same loss and gradients as the fused attention, on a batch with padding."""
    from superscaler_b200.runtime.trainer import Trainer
    plan = tiny_bert_plan(**dict(KW, micro_bs=8))
    b = _batch(seed=4)
    assert int(b["enc_lens"].min()) < KW["seq"]
    runs = []
    for fuse in (True, False):
        t = Trainer(plan, device="cpu", model_overrides=OV, lr_warmup_steps=0, fuse=fuse, seed=7)
        loss = t.forward_backward(t.to_device(b))
        t._fold_autograd_grads()
        runs.append((float(loss), t.store.grad.clone()))
    (la, ga), (lb, gb) = runs
    assert abs(la - lb) < 2e-3 * abs(la)
    assert float((ga - gb).norm()) < 2e-2 * float(ga.norm())
