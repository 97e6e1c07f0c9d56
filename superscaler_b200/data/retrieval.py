"""Open-retrieval evidence index: embed every block of an evidence file once, keep (block id -> embedding) in shards,
merge them, and answer maximum-inner-product queries.

Reference counterparts (inherited from Megatron's REALM / ORQA code, unused by the op-list models):
runtime/megatron/indexer.py (IndexBuilder: one pass over the evidence data, one shard per data-parallel rank, rank 0
merges), runtime/megatron/data/realm_index.py (OpenRetreivalDataStore, FaissMIPSIndex),
runtime/megatron/data/orqa_wiki_dataset.py (tab-separated evidence rows -> [CLS] title [SEP] text [SEP]).

Differences by design:
  * shards and the merged store are `.npz` files (int64 ids, fp16 embeddings), not pickles;
  * the index is an exact chunked matrix product on the GPU (or CPU) instead of FAISS: 21 M blocks x 128 dims in
    fp16 are 5.4 GB, which fits a B200 many times over, and a flat FAISS index is exact as well;
  * the embedder is any callable (token ids, padding mask) -> [n, d]; `HashedBagOfWords` is a dependency-free one
    so that the command line works end to end without a trained encoder.

    python -m superscaler_b200.data.retrieval build --evidence blocks.tsv --vocab vocab.txt --out index_dir
    python -m superscaler_b200.data.retrieval query --index index_dir --vocab vocab.txt --text "who ..." --topk 5
(`build` under torch.distributed.run: one shard per rank, rank 0 merges.)
"""
from __future__ import annotations

import argparse
import csv
import glob
import os
import sys
from typing import Callable, Iterator, List, Optional, Tuple

import numpy as np
import torch


# ---- evidence rows ------------------------------------------------------------------------------------
class EvidenceBlocks:
    """Rows `id <tab> text <tab> title` (a header line whose first field is not a number is skipped).  Item i is
    (row id, token ids, padding mask, token types): [CLS] title [SEP] text [SEP], cut and padded to `seq_length`."""

    def __init__(self, path: str, encode: Callable[[str], List[int]], cls_id: int, sep_id: int, pad_id: int,
                 seq_length: int = 256):
        self.encode, self.cls, self.sep, self.pad, self.seq = encode, cls_id, sep_id, pad_id, seq_length
        self.rows: List[Tuple[int, str, str]] = []
        csv.field_size_limit(sys.maxsize)
        with open(path, newline="", encoding="utf-8") as f:
            for rec in csv.reader(f, delimiter="\t"):
                if not rec:
                    continue
                try:
                    rid = int(rec[0])
                except ValueError:
                    continue
                self.rows.append((rid, rec[1] if len(rec) > 1 else "", rec[2] if len(rec) > 2 else ""))

    def __len__(self) -> int:
        return len(self.rows)

    def __getitem__(self, i: int):
        rid, text, title = self.rows[i]
        t, x = self.encode(title), self.encode(text)
        room = self.seq - 3
        t = t[:room]
        x = x[:max(0, room - len(t))]
        ids = [self.cls] + t + [self.sep] + x + [self.sep]
        types = [0] * (len(t) + 2) + [1] * (len(x) + 1)
        n = len(ids)
        ids += [self.pad] * (self.seq - n)
        types += [0] * (self.seq - n)
        mask = [1] * n + [0] * (self.seq - n)
        return rid, np.asarray(ids, np.int64), np.asarray(mask, np.bool_), np.asarray(types, np.int64)

    def batches(self, batch_size: int, rank: int = 0, world: int = 1) -> Iterator[tuple]:
        """Batches of the rows this rank owns: batch b of the file goes to rank b % world."""
        nb = (len(self) + batch_size - 1) // batch_size
        for b in range(rank, nb, world):
            items = [self[i] for i in range(b * batch_size, min(len(self), (b + 1) * batch_size))]
            yield (torch.tensor([it[0] for it in items], dtype=torch.int64),
                   torch.from_numpy(np.stack([it[1] for it in items])),
                   torch.from_numpy(np.stack([it[2] for it in items])),
                   torch.from_numpy(np.stack([it[3] for it in items])))


class HashedBagOfWords:
    """[n, dim] embeddings from token counts through a fixed random projection (seeded): equal texts get equal
    vectors, texts that share tokens get a positive inner product.  Stands in for a trained block encoder."""

    def __init__(self, vocab_size: int, dim: int = 128, seed: int = 0, device="cpu"):
        g = torch.Generator().manual_seed(seed)
        self.table = (torch.randn(vocab_size, dim, generator=g) / dim ** 0.5).to(device)

    def __call__(self, ids: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
        e = self.table[ids.to(self.table.device)] * mask.to(self.table.device)[..., None].to(self.table.dtype)
        v = e.sum(1)
        return v / v.norm(dim=-1, keepdim=True).clamp(min=1e-6)


# ---- store --------------------------------------------------------------------------------------------
class EmbeddingStore:
    """(block id -> embedding) collected by one rank, saved as a shard, merged by rank 0."""

    def __init__(self, directory: str, rank: int = 0):
        self.dir, self.rank = directory, rank
        self.ids: List[np.ndarray] = []
        self.emb: List[np.ndarray] = []

    def add(self, ids: torch.Tensor, embeddings: torch.Tensor) -> None:
        assert ids.shape[0] == embeddings.shape[0]
        self.ids.append(ids.detach().cpu().numpy().astype(np.int64))
        self.emb.append(embeddings.detach().float().cpu().numpy().astype(np.float16))

    def _shard_path(self, rank: int) -> str:
        return os.path.join(self.dir, "shards", f"{rank}.npz")

    def save_shard(self) -> str:
        os.makedirs(os.path.join(self.dir, "shards"), exist_ok=True)
        ids = np.concatenate(self.ids) if self.ids else np.zeros((0,), np.int64)
        emb = np.concatenate(self.emb) if self.emb else np.zeros((0, 0), np.float16)
        tmp = self._shard_path(self.rank) + ".tmp.npz"
        np.savez(tmp, ids=ids, emb=emb)
        os.replace(tmp, self._shard_path(self.rank))
        return self._shard_path(self.rank)

    def merge_shards_and_save(self, world: int) -> str:
        """All `world` shards must be present (a missing one is an error, not a smaller index); duplicate ids are
        refused.  Rows are stored in id order."""
        parts = []
        for r in range(world):
            p = self._shard_path(r)
            if not os.path.exists(p):
                raise FileNotFoundError(f"shard of rank {r} is missing: {p}")
            z = np.load(p)
            if z["ids"].shape[0]:
                parts.append((z["ids"], z["emb"]))
        ids = np.concatenate([a for a, _ in parts])
        emb = np.concatenate([b for _, b in parts])
        if np.unique(ids).shape[0] != ids.shape[0]:
            raise ValueError("the shards contain a block id more than once")
        order = np.argsort(ids, kind="stable")
        out = os.path.join(self.dir, "store.npz")
        np.savez(out + ".tmp.npz", ids=ids[order], emb=emb[order])
        os.replace(out + ".tmp.npz", out)
        for p in glob.glob(os.path.join(self.dir, "shards", "*.npz")):
            os.remove(p)
        return out

    @staticmethod
    def load(directory: str) -> Tuple[np.ndarray, np.ndarray]:
        z = np.load(os.path.join(directory, "store.npz"))
        return z["ids"], z["emb"]


# ---- index --------------------------------------------------------------------------------------------
class MIPSIndex:
    """Exact maximum-inner-product search: scores = queries x blocks^T in chunks of blocks, running top-k."""

    def __init__(self, ids: np.ndarray, embeddings: np.ndarray, device="cpu", chunk: int = 1 << 20):
        self.ids = torch.from_numpy(np.ascontiguousarray(ids))
        dt = torch.float16 if str(device).startswith("cuda") else torch.float32
        self.emb = torch.from_numpy(np.ascontiguousarray(embeddings)).to(device=device, dtype=dt)
        self.chunk = chunk

    def search(self, queries: torch.Tensor, topk: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """([n, topk] scores in descending order, [n, topk] block ids)."""
        q = queries.to(device=self.emb.device, dtype=self.emb.dtype)
        k = min(topk, self.emb.shape[0])
        best_s = torch.full((q.shape[0], 0), 0.0, device=q.device)
        best_i = torch.zeros((q.shape[0], 0), dtype=torch.int64, device=q.device)
        for c0 in range(0, self.emb.shape[0], self.chunk):
            s = (q @ self.emb[c0:c0 + self.chunk].t()).float()
            cs, ci = s.topk(min(k, s.shape[1]), dim=1)
            best_s = torch.cat([best_s, cs], 1)
            best_i = torch.cat([best_i, ci + c0], 1)
            best_s, sel = best_s.topk(min(k, best_s.shape[1]), dim=1)
            best_i = best_i.gather(1, sel)
        return best_s.cpu(), self.ids[best_i.cpu()]


# ---- builder ------------------------------------------------------------------------------------------
def build_index(blocks: EvidenceBlocks, embed: Callable[[torch.Tensor, torch.Tensor], torch.Tensor], directory: str,
                batch_size: int = 128, rank: int = 0, world: int = 1, barrier: Optional[Callable[[], None]] = None,
                log_interval: int = 0) -> Optional[str]:
    """One pass over the evidence rows: every rank embeds its batches and writes a shard; after `barrier()` rank 0
    merges the shards and returns the path of the merged store (other ranks return None)."""
    store = EmbeddingStore(directory, rank)
    with torch.no_grad():
        for n, (rid, ids, mask, _types) in enumerate(blocks.batches(batch_size, rank, world), 1):
            store.add(rid, embed(ids, mask))
            if log_interval and rank == 0 and n % log_interval == 0:
                print(f"Batch {n:10d} | Total {n * batch_size * world:10d}", flush=True)
    store.save_shard()
    if barrier is not None:
        barrier()
    return store.merge_shards_and_save(world) if rank == 0 else None


def _encoder(vocab_path: str):
    from ..tokenizer.wordpiece import WordPieceEncoder, load_vocab
    vocab = load_vocab(vocab_path)
    enc = WordPieceEncoder(vocab)
    return enc, vocab


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="cmd", required=True)
    b = sub.add_parser("build")
    b.add_argument("--evidence", required=True), b.add_argument("--vocab", required=True)
    b.add_argument("--out", required=True), b.add_argument("--seq-length", type=int, default=256)
    b.add_argument("--indexer-batch-size", type=int, default=128), b.add_argument("--indexer-log-interval", type=int, default=1000)
    b.add_argument("--dim", type=int, default=128)
    q = sub.add_parser("query")
    q.add_argument("--index", required=True), q.add_argument("--vocab", required=True)
    q.add_argument("--text", required=True, nargs="+"), q.add_argument("--topk", type=int, default=5)
    q.add_argument("--seq-length", type=int, default=256), q.add_argument("--dim", type=int, default=128)
    a = ap.parse_args(argv)
    enc, vocab = _encoder(a.vocab)
    device = "cuda" if torch.cuda.is_available() else "cpu"
    embed = HashedBagOfWords(len(vocab), a.dim, device=device)
    if a.cmd == "build":
        import torch.distributed as dist
        rank, world, barrier = 0, 1, None
        if "RANK" in os.environ:
            dist.init_process_group("nccl" if torch.cuda.is_available() else "gloo")
            rank, world, barrier = dist.get_rank(), dist.get_world_size(), dist.barrier
        blocks = EvidenceBlocks(a.evidence, enc.encode, vocab["[CLS]"], vocab["[SEP]"], vocab["[PAD]"], a.seq_length)
        out = build_index(blocks, embed, a.out, a.indexer_batch_size, rank, world, barrier, a.indexer_log_interval)
        if out:
            print(f"wrote {out} ({len(blocks)} blocks)")
        if barrier is not None:
            dist.barrier()
            dist.destroy_process_group()
        return
    ids, emb = EmbeddingStore.load(a.index)
    index = MIPSIndex(ids, emb, device=device)
    rows = []
    for text in a.text:
        t = [vocab["[CLS]"]] + enc.encode(text)[:a.seq_length - 2] + [vocab["[SEP]"]]
        rows.append(t + [vocab["[PAD]"]] * (a.seq_length - len(t)))
    tok = torch.tensor(rows, dtype=torch.int64)
    scores, found = index.search(embed(tok, tok != vocab["[PAD]"]), a.topk)
    for text, s, f in zip(a.text, scores, found):
        print(text, "->", ", ".join(f"{int(i)} ({float(v):.3f})" for i, v in zip(f, s)))


if __name__ == "__main__":
    main()
