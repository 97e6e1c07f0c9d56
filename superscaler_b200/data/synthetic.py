"""Synthetic batches of the shapes the benchmarks name, generated on the host from a seed into pinned
memory (the reference draws its batches on the device inside get_batch: runtime/pretrain_gpt.py:50-62,
runtime/pretrain_t5.py:72-86, runtime/pretrain_resnet.py:48-60)."""
from __future__ import annotations

from typing import Dict, Iterator

import torch


def _pin(t: torch.Tensor) -> torch.Tensor:
    return t.pin_memory() if torch.cuda.is_available() else t


def gpt_batch(global_bs: int, seq: int, vocab: int, seed: int) -> Dict[str, torch.Tensor]:
    """Token ids uniform over [0, vocab); labels are the ids shifted by one; every position counts."""
    g = torch.Generator().manual_seed(seed)
    tokens = torch.randint(0, vocab, (global_bs, seq + 1), generator=g, dtype=torch.int64)
    return {"ids": _pin(tokens[:, :-1].contiguous()), "labels": _pin(tokens[:, 1:].contiguous())}


def t5_batch(global_bs: int, enc_seq: int, dec_seq: int, vocab: int, seed: int) -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    enc = torch.randint(0, vocab, (global_bs, enc_seq), generator=g, dtype=torch.int64)
    dec = torch.randint(0, vocab, (global_bs, dec_seq + 1), generator=g, dtype=torch.int64)
    return {"ids": _pin(enc), "dec_ids": _pin(dec[:, :-1].contiguous()), "labels": _pin(dec[:, 1:].contiguous())}


def bert_batch(global_bs: int, seq: int, vocab: int, seed: int, masked_fraction: float = 0.15) -> Dict[str, torch.Tensor]:
    """Two-segment samples of random length: token ids, token types (0 / 1), the number of real tokens per sample,
    masked-LM labels at a random 15 % of the real positions (-1 elsewhere, loss_mask 1 there) and a random
    sentence-order flag."""
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(5, vocab, (global_bs, seq), generator=g, dtype=torch.int64)
    lens = torch.randint(max(2, seq // 2), seq + 1, (global_bs,), generator=g, dtype=torch.int32)
    cut = (lens.to(torch.float32) * (0.25 + 0.5 * torch.rand(global_bs, generator=g))).to(torch.int64).clamp(min=1)
    pos = torch.arange(seq)[None, :]
    real = pos < lens[:, None]
    types = ((pos >= cut[:, None]) & real).to(torch.int64)
    ids = torch.where(real, ids, torch.zeros_like(ids))                      # 0 = padding id
    masked = (torch.rand(global_bs, seq, generator=g) < masked_fraction) & real
    labels = torch.where(masked, ids, torch.full_like(ids, -1))
    ids = torch.where(masked, torch.full_like(ids, 4), ids)                   # 4 = [MASK]
    nsp = torch.randint(0, 2, (global_bs,), generator=g, dtype=torch.int64)
    return {"ids": _pin(ids), "types": _pin(types), "enc_lens": _pin(lens), "labels": _pin(labels),
            "loss_mask": _pin(masked.to(torch.float32)), "nsp": _pin(nsp)}


def resnet_batch(global_bs: int, image: int, classes: int, seed: int, dtype=torch.bfloat16) -> Dict[str, torch.Tensor]:
    """N(0,1) images in NHWC and uniform labels."""
    g = torch.Generator().manual_seed(seed)
    img = torch.randn((global_bs, image, image, 3), generator=g, dtype=torch.float32).to(dtype)
    lab = torch.randint(0, classes, (global_bs,), generator=g, dtype=torch.int64)
    return {"images": _pin(img), "labels": _pin(lab)}


def batches(kind: str, steps: int, seed: int = 1234, **kw) -> Iterator[Dict[str, torch.Tensor]]:
    fn = {"gpt": gpt_batch, "t5": t5_batch, "resnet": resnet_batch, "bert": bert_batch}[kind]
    for i in range(steps):
        yield fn(seed=seed + i, **kw)
