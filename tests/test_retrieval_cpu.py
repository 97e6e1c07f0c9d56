"""Evidence index: row encoding, shards written by two gloo ranks and merged by rank 0, exact top-k search, and the
failure cases of the merge (a missing shard, a repeated block id)."""
import os

import numpy as np
import pytest
import torch

from superscaler_b200.data import retrieval as R
from dist_utils import run_ranks

WORDS = "alpha beta gamma delta epsilon zeta eta theta iota kappa lambda mu nu xi omicron pi rho sigma tau".split()
VOCAB = {w: i for i, w in enumerate(["[PAD]", "[CLS]", "[SEP]", "[UNK]"] + WORDS)}


def _encode(text):
    return [VOCAB.get(w, VOCAB["[UNK]"]) for w in text.split()]


def _write_tsv(path, n=53):
    rs = np.random.RandomState(0)
    with open(path, "w", encoding="utf-8") as f:
        f.write("id\ttext\ttitle\n")
        for i in range(n):
            text = " ".join(rs.choice(WORDS, size=rs.randint(3, 12)))
            f.write(f"{1000 + i}\t{text}\t{WORDS[i % len(WORDS)]}\n")


def _blocks(path, seq=16):
    return R.EvidenceBlocks(path, _encode, VOCAB["[CLS]"], VOCAB["[SEP]"], VOCAB["[PAD]"], seq)


def test_rows_are_cls_title_sep_text_sep_padded(tmp_path):
    p = str(tmp_path / "ev.tsv")
    _write_tsv(p)
    b = _blocks(p)
    assert len(b) == 53                                     # the header line is skipped
    rid, ids, mask, types = b[0]
    assert rid == 1000 and ids.shape == (16,) and ids[0] == VOCAB["[CLS]"] and ids[2] == VOCAB["[SEP]"]
    n = int(mask.sum())
    assert ids[n - 1] == VOCAB["[SEP]"] and (ids[n:] == VOCAB["[PAD]"]).all()
    assert list(types[:3]) == [0, 0, 0] and types[3] == 1 and (types[n:] == 0).all()
    long_b = R.EvidenceBlocks(p, lambda t: _encode(t) * 9, 1, 2, 0, 16)
    assert int(long_b[0][2].sum()) == 16                     # cut to the sequence length, still ends with [SEP]
    assert long_b[0][1][15] == 2


def _build_worker(rank, world, tsv, out):
    import torch.distributed as dist
    blocks = _blocks(tsv)
    embed = R.HashedBagOfWords(len(VOCAB), 32, seed=1)
    R.build_index(blocks, embed, out, batch_size=8, rank=rank, world=world, barrier=dist.barrier)


def test_two_ranks_build_one_index_and_search_is_exact(tmp_path):
    tsv, out = str(tmp_path / "ev.tsv"), str(tmp_path / "index")
    _write_tsv(tsv)
    run_ranks(_build_worker, 2, tsv, out)
    ids, emb = R.EmbeddingStore.load(out)
    assert list(ids) == list(range(1000, 1053)) and emb.shape == (53, 32) and emb.dtype == np.float16
    assert not os.listdir(os.path.join(out, "shards"))       # shards are removed after the merge
    # one rank alone writes the same store
    solo = str(tmp_path / "solo")
    R.build_index(_blocks(tsv), R.HashedBagOfWords(len(VOCAB), 32, seed=1), solo, batch_size=8)
    ids1, emb1 = R.EmbeddingStore.load(solo)
    assert np.array_equal(ids, ids1) and np.array_equal(emb, emb1)
    index = R.MIPSIndex(ids, emb, chunk=10)                  # several chunks, running top-k across them
    q = torch.from_numpy(emb[[5, 17, 40]].astype(np.float32))
    scores, found = index.search(q, 4)
    ref = q @ torch.from_numpy(emb.astype(np.float32)).t()
    rs, ri = ref.topk(4, dim=1)
    assert torch.allclose(scores, rs, atol=1e-5) and torch.equal(found, torch.from_numpy(ids)[ri])
    assert list(found[:, 0]) == [1005, 1017, 1040]           # a block's own embedding is its best match


def test_merge_refuses_a_missing_shard_and_a_repeated_id(tmp_path):
    d = str(tmp_path / "idx")
    s0 = R.EmbeddingStore(d, 0)
    s0.add(torch.tensor([1, 2]), torch.randn(2, 4))
    s0.save_shard()
    with pytest.raises(FileNotFoundError):
        s0.merge_shards_and_save(world=2)
    s1 = R.EmbeddingStore(d, 1)
    s1.add(torch.tensor([2, 3]), torch.randn(2, 4))
    s1.save_shard()
    with pytest.raises(ValueError):
        s0.merge_shards_and_save(world=2)


def test_command_line_builds_and_queries(tmp_path, capsys):
    tsv, out, vocab = str(tmp_path / "ev.tsv"), str(tmp_path / "index"), str(tmp_path / "vocab.txt")
    _write_tsv(tsv)
    with open(vocab, "w") as f:
        f.write("\n".join(VOCAB) + "\n")
    R.main(["build", "--evidence", tsv, "--vocab", vocab, "--out", out, "--seq-length", "16", "--dim", "32",
            "--indexer-batch-size", "8"])
    R.main(["query", "--index", out, "--vocab", vocab, "--text", "alpha beta gamma", "--topk", "3", "--seq-length", "16",
            "--dim", "32"])
    assert "alpha beta gamma ->" in capsys.readouterr().out
