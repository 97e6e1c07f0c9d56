"""Flat parameter storage of one pipeline stage.

Every parameter of a stage is a view into five flat, equally laid out buffers: fp32 master values,
fp32 main gradients, two fp32 Adam moments and the bf16 model copy the GEMM kernels read.  One fused
optimizer launch updates the whole stage, and GEMM wgrad kernels accumulate directly into the
main-gradient views (``param.main_grad``).  Parameters with weight decay come first so the kernel needs
only one split index.

Plays the role of the reference's Float16OptimizerWithFloat16Params bookkeeping
(runtime/megatron/optimizer/optimizer.py:232-279) and of LocalDDP's contiguous gradient buffer
(runtime/megatron/model/distributed.py:122-169), which the reference refuses in resharding stages; here
the buffer is always flat and per-(tp, dp) bucket ranges are recorded for the data-parallel reduction.
"""
from __future__ import annotations

import zlib
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch


@dataclass
class ParamSpec:
    name: str
    shape: Tuple[int, ...]            # local (sharded) shape
    init: str                         # "normal" | "zeros" | "ones" | "kaiming"
    std: float = 0.02
    weight_decay: bool = True
    fp32: bool = False                # the model reads the fp32 master directly (LayerNorm / BatchNorm)
    full_shape: Optional[Tuple[int, ...]] = None   # unsharded shape, for TP-invariant initialisation
    shard_dim: Optional[int] = None   # dimension split across the TP group
    tp: int = 1
    tp_rank: int = 0
    dp: int = 1
    seed_key: str = ""                # parameters with equal seed_key and full_shape start identical
    shared_key: Optional[str] = None  # tied weights (e.g. word embeddings used by the LM head)


def _align(n: int, a: int = 128) -> int:
    return (n + a - 1) // a * a


class ParamStore:
    def __init__(self, device, base_seed: int = 1234):
        self.device = torch.device(device)
        self.base_seed = base_seed
        self.specs: List[ParamSpec] = []
        self.params: Dict[str, torch.nn.Parameter] = {}
        self.offsets: Dict[str, Tuple[int, int]] = {}
        self.master = self.grad = self.exp_avg = self.exp_avg_sq = self.model16 = None
        self.wd_end = 0
        self.total = 0
        self._shared: Dict[Tuple[str, int], str] = {}   # (shared key, tensor-parallel degree) -> parameter name
        self.grad_allocator = None      # optional: numel -> (tensor, owner) for a peer-mapped gradient buffer
        self.symm_grad = None
        self.model16_allocator = None   # optional: numel -> peer-mapped bf16 model buffer (sharded optimizer step)
        self.symm_model16 = None

    def declare(self, spec: ParamSpec) -> str:
        """Registers a parameter; tied parameters (same shared_key AND the same tensor-parallel degree, hence the
        same shard) resolve to the first declaration.  Ops of one stage that share a weight under different
        degrees keep a copy each; runtime/tied.py keeps such copies equal, as it does across stages."""
        if spec.shared_key is not None:
            k = (spec.shared_key, spec.tp)
            if k in self._shared:
                return self._shared[k]
            self._shared[k] = spec.name
        self.specs.append(spec)
        return spec.name

    def _init_full(self, spec: ParamSpec) -> torch.Tensor:
        shape = spec.full_shape or spec.shape
        if spec.init == "zeros":
            return torch.zeros(shape, dtype=torch.float32, device=self.device)
        if spec.init == "ones":
            return torch.ones(shape, dtype=torch.float32, device=self.device)
        gen = torch.Generator(device=self.device)
        gen.manual_seed((self.base_seed * 1000003 + zlib.crc32((spec.seed_key or spec.name).encode())) % (2 ** 63))
        w = torch.empty(shape, dtype=torch.float32, device=self.device)
        if spec.init == "normal":
            w.normal_(0.0, spec.std, generator=gen)
        elif spec.init == "kaiming":
            fan_in = 1
            for d in shape[1:]:
                fan_in *= d
            w.normal_(0.0, (2.0 / fan_in) ** 0.5, generator=gen)
        else:
            raise ValueError(spec.init)
        return w

    def materialize(self) -> None:
        ordered = [s for s in self.specs if s.weight_decay] + [s for s in self.specs if not s.weight_decay]
        off = 0
        for s in ordered:
            n = 1
            for d in s.shape:
                n *= d
            self.offsets[s.name] = (off, n)
            off += _align(n)
            if s.weight_decay:
                self.wd_end = off
        self.total = max(off, 128)
        f32 = dict(dtype=torch.float32, device=self.device)
        self.master = torch.zeros(self.total, **f32)
        if self.grad_allocator is not None:
            self.symm_grad = self.grad_allocator(self.total)
            self.grad = self.symm_grad.tensor
        else:
            self.grad = torch.zeros(self.total, **f32)
        self.exp_avg = torch.zeros(self.total, **f32)
        self.exp_avg_sq = torch.zeros(self.total, **f32)
        if self.model16_allocator is not None:
            self.symm_model16 = self.model16_allocator(self.total)
            self.model16 = self.symm_model16.tensor
        else:
            self.model16 = torch.zeros(self.total, dtype=torch.bfloat16, device=self.device)
        for s in ordered:
            off, n = self.offsets[s.name]
            full = self._init_full(s)
            if s.full_shape is not None and s.shard_dim is not None and s.tp > 1:
                full = full.chunk(s.tp, dim=s.shard_dim)[s.tp_rank]
            # master values start as the bf16-rounded initial weights so both copies agree exactly
            rounded = full.reshape(-1).to(torch.bfloat16)
            if s.fp32:
                self.master[off:off + n].copy_(full.reshape(-1))
            else:
                self.master[off:off + n].copy_(rounded.float())
            self.model16[off:off + n].copy_(rounded)
            del full
            data = (self.master if s.fp32 else self.model16)[off:off + n].view(s.shape)
            p = torch.nn.Parameter(data, requires_grad=True)
            p.main_grad = self.grad[off:off + n].view(s.shape)
            p.spec = s
            self.params[s.name] = p

    def shared_name(self, key: str, tp: int) -> Optional[str]:
        return self._shared.get((key, tp))

    def __getitem__(self, name: str) -> torch.nn.Parameter:
        return self.params[name]

    def zero_grad(self) -> None:
        self.grad.zero_()

    def buckets_by_dp(self) -> Dict[Tuple[int, int], List[Tuple[int, int]]]:
        """(tp, dp) -> [(offset, length)] contiguous ranges of the gradient buffer owned by ops with those degrees."""
        out: Dict[Tuple[int, int], List[Tuple[int, int]]] = {}
        for s in self.specs:
            off, n = self.offsets[s.name]
            key = (s.tp, s.dp)
            rng = out.setdefault(key, [])
            if rng and rng[-1][0] + rng[-1][1] == off:
                rng[-1] = (rng[-1][0], rng[-1][1] + _align(n))
            else:
                rng.append((off, _align(n)))
        for key in out:
            merged: List[Tuple[int, int]] = []
            for off, n in sorted(out[key]):
                if merged and merged[-1][0] + merged[-1][1] == off:
                    merged[-1] = (merged[-1][0], merged[-1][1] + n)
                else:
                    merged.append((off, n))
            out[key] = merged
        return out

    def state_dict(self) -> Dict[str, torch.Tensor]:
        return {name: (self.master[o:o + n].view(self.params[name].shape).clone())
                for name, (o, n) in self.offsets.items()}

    def load_state_dict(self, sd: Dict[str, torch.Tensor]) -> None:
        for name, (o, n) in self.offsets.items():
            v = sd[name].to(self.device, torch.float32).reshape(-1)
            self.master[o:o + n].copy_(v)
            self.model16[o:o + n].copy_(v.to(torch.bfloat16))
