"""Broadcast of a batch dictionary from one rank of a group to the others, for loaders that read real data on a
single rank per tensor-parallel group (reference: broadcast_data, runtime/megatron/mpu/data.py:76-117).

All tensors of one dtype travel as ONE flat buffer; their shapes go first in a small int64 message, so the
receivers need not know them in advance.
"""
from __future__ import annotations

from typing import Dict, Optional, Sequence

import torch
import torch.distributed as dist

_MAX_DIMS = 5


def broadcast_batch(keys: Sequence[str], batch: Optional[Dict[str, torch.Tensor]], dtype: torch.dtype, src: int,
                    group=None, device=None) -> Dict[str, torch.Tensor]:
    """`batch` is read on rank `src` only (global rank, member of `group`); every rank returns the same dict."""
    rank = dist.get_rank()
    device = torch.device(device) if device is not None else torch.device("cpu")
    sizes = torch.zeros(len(keys) * _MAX_DIMS, dtype=torch.int64, device=device)
    if rank == src:
        for i, k in enumerate(keys):
            t = batch[k]
            assert t.dim() <= _MAX_DIMS and t.dtype == dtype, f"{k}: at most {_MAX_DIMS} dims of dtype {dtype}"
            for j, d in enumerate(t.shape):
                sizes[i * _MAX_DIMS + j] = d
    dist.broadcast(sizes, src, group=group)
    shapes = []
    for i in range(len(keys)):
        dims = sizes[i * _MAX_DIMS:(i + 1) * _MAX_DIMS].tolist()
        while dims and dims[-1] == 0:
            dims.pop()
        shapes.append(tuple(int(d) for d in dims))
    counts = [int(torch.Size(s).numel()) for s in shapes]
    if rank == src:
        flat = torch.cat([batch[k].reshape(-1).to(device) for k in keys])
    else:
        flat = torch.empty(sum(counts), dtype=dtype, device=device)
    dist.broadcast(flat, src, group=group)
    out, at = {}, 0
    for k, s, n in zip(keys, shapes, counts):
        out[k] = flat[at:at + n].view(s)
        at += n
    return out
