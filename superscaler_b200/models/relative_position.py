"""T5 relative-position attention bias.

The bias added to the attention scores of head h for query i and key j depends on the signed distance j - i
alone: it is row bucket(j - i) of a learned [buckets, heads] table.  Buckets are exact for small distances and
logarithmic up to `max_distance` (half the buckets per direction when the attention looks both ways).  Because of
that, everything a kernel needs is a per-head TABLE OVER THE DISTANCE with sq + sk - 1 entries
(`distance_table`); the full [heads, sq, sk] bias (`bias_from_table`) is only materialised by the reference path.
The reference's T5 has no such bias (learned absolute positions, runtime/megatron/model/flex_t5.py:23-42); the
benchmark's T5 definition does.
"""
from __future__ import annotations

import math

import torch


def relative_position_bucket(distance: torch.Tensor, bidirectional: bool, num_buckets: int = 32,
                             max_distance: int = 128) -> torch.Tensor:
    """Bucket index of key_position - query_position (int64 tensor of any shape)."""
    d = distance.to(torch.int64)
    if bidirectional:
        num_buckets //= 2
        offset = (d > 0).to(torch.int64) * num_buckets      # keys after the query use the upper half
        d = d.abs()
    else:
        offset = torch.zeros_like(d)
        d = (-d).clamp(min=0)                               # only keys at or before the query are told apart
    exact = num_buckets // 2
    small = d < exact
    # distances exact .. max_distance share the remaining buckets on a logarithmic scale
    scaled = exact + (torch.log(d.clamp(min=1).float() / exact) / math.log(max_distance / exact)
                      * (num_buckets - exact)).to(torch.int64)
    scaled = scaled.clamp(max=num_buckets - 1)
    return offset + torch.where(small, d, scaled)


_BUCKETS_OF_DISTANCE = {}


def buckets_of_distances(sq: int, sk: int, bidirectional: bool, num_buckets: int, max_distance: int,
                         device) -> torch.Tensor:
    """Bucket of every distance -(sq - 1) .. sk - 1, computed once per geometry and device (every layer of every
    micro-batch asks for the same sq + sk - 1 integers)."""
    key = (sq, sk, bool(bidirectional), num_buckets, max_distance, str(device))
    idx = _BUCKETS_OF_DISTANCE.get(key)
    if idx is None:
        dist = torch.arange(-(sq - 1), sk, device=device)
        idx = relative_position_bucket(dist, bidirectional, num_buckets, max_distance)
        _BUCKETS_OF_DISTANCE[key] = idx
    return idx


def distance_table(weight: torch.Tensor, sq: int, sk: int, bidirectional: bool, num_buckets: int = 32,
                   max_distance: int = 128) -> torch.Tensor:
    """weight [heads, buckets] -> [heads, sq + sk - 1]; column c holds the bias of distance c - (sq - 1)."""
    return weight[:, buckets_of_distances(sq, sk, bidirectional, num_buckets, max_distance, weight.device)]


def bias_from_table(table: torch.Tensor, sq: int, sk: int) -> torch.Tensor:
    """[heads, sq + sk - 1] -> [heads, sq, sk] with bias[h, i, j] = table[h, j - i + sq - 1]."""
    idx = torch.arange(sk, device=table.device)[None, :] - torch.arange(sq, device=table.device)[:, None] + (sq - 1)
    return table[:, idx]
