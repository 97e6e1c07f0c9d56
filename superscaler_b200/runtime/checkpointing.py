"""Checkpoint save / load in the Megatron v3.0 directory layout used by the reference
(runtime/megatron/checkpointing.py:83-170):

    {save}/latest_checkpointed_iteration.txt
    {save}/iter_{0000000}/mp_rank_{tp:02d}[_{pp:03d}]/model_optim_rng.pt

with the keys ``args, checkpoint_version (3.0), iteration, model, optimizer, lr_scheduler, rng`` and, in
addition, ``plan`` (the plan JSON the run used) and ``op_names`` (index -> op name), so a checkpoint written under
one plan can be re-assembled under another.  Only data-parallel rank 0 of each (stage, tp rank) writes.  Parameter
names inside ``model`` follow the reference's ``language_model.ops.{i}.{module}.{weight|bias}`` convention with
i = the op's index inside its stage (runtime/megatron/model/flex_model.py:378); with interleaving a stage's later
chunks continue the numbering from the global op indices (i = global index - first op of the stage's chunk 0).

`merge_tp_shards` / `load_under_plan` rebuild full (unsharded) tensors from the tp shards of a checkpoint and
re-slice them for a new plan.
"""
from __future__ import annotations

import os
import random
from typing import Dict, Optional

import numpy as np
import torch

from ..ops import functional as F

TRACKER = "latest_checkpointed_iteration.txt"


class CheckpointError(RuntimeError):
    """A checkpoint file is missing, truncated or unreadable; the message names the file."""


def _load_file(path: str):
    try:
        return torch.load(path, map_location="cpu", weights_only=False)
    except Exception as e:  # noqa: BLE001 - zip / pickle errors of a damaged shard
        raise CheckpointError(f"cannot read checkpoint shard {path}: {type(e).__name__}: {e}") from e


def checkpoint_dir(root: str, iteration, tp_rank: int, pp_rank: int, pp_size: int) -> str:
    tag = "release" if iteration == "release" else "iter_{:07d}".format(iteration)
    sub = "mp_rank_{:02d}".format(tp_rank) if pp_size == 1 else "mp_rank_{:02d}_{:03d}".format(tp_rank, pp_rank)
    return os.path.join(root, tag, sub)


def _local_names(trainer) -> Dict[str, str]:
    """store name (ops.{global index}.x) -> checkpoint name (language_model.ops.{local index}.x)."""
    lo = trainer.stage_bounds[trainer.pstate.stage][0]
    out = {}
    for name in trainer.store.params:
        _, idx, rest = name.split(".", 2)
        out[name] = f"language_model.ops.{int(idx) - lo}.{rest}"
    return out


def _buffers(trainer) -> Dict[str, torch.Tensor]:
    """Non-parameter state of the ops (BatchNorm running statistics), keyed like the parameters of their op."""
    lo = trainer.stage_bounds[trainer.pstate.stage][0]
    out = {}
    for op in trainer.stage.raw_ops:
        for owner in (op, getattr(op, "bn_op", None)):
            if owner is not None and getattr(owner, "run_mean", None) is not None:
                base = f"language_model.ops.{owner.info.index - lo}.{owner.key}"
                out[base + ".running_mean"], out[base + ".running_var"] = owner.run_mean, owner.run_var
    return out


def _shard_of(trainer):
    """(does this rank write, shard number in the directory name).  A stage whose ops all use one tensor-parallel
    degree is written by the data-parallel rank 0 of every tensor-parallel rank, as in the reference
    (runtime/megatron/checkpointing.py:121).  In a stage that mixes degrees a rank can hold the only copy of one
    op's shard while being a replica for another op, so every rank writes, numbered by its position in the stage."""
    ps = trainer.pstate
    first = trainer.infos[0]
    pl = ps.placement(first.tp, first.dp)
    if len({i.tp for i in trainer.infos}) == 1:
        return pl.dp_rank == 0, pl.tp_rank
    return True, ps.local_rank_in_stage


def save_checkpoint(trainer, root: str, iteration: Optional[int] = None) -> Optional[str]:
    it = trainer.iteration if iteration is None else iteration
    ps = trainer.pstate
    if hasattr(trainer, "check_device_status"):
        trainer.check_device_status()        # never write weights that a timed-out kernel may have corrupted
    if hasattr(trainer.optimizer, "sync_replicas"):
        trainer.optimizer.sync_replicas()    # collective: the slices other ranks own after sharded optimizer steps
    writes, shard = _shard_of(trainer)
    path = None
    if writes:
        d = checkpoint_dir(root, it, shard, ps.stage, ps.num_stages)
        os.makedirs(d, exist_ok=True)
        names = _local_names(trainer)
        model = {names[k]: v.cpu() for k, v in trainer.store.state_dict().items()}
        sd = {
            "args": {"plan": trainer.plan, "model_name": trainer.model_name},
            "checkpoint_version": 3.0,
            "iteration": it,
            "model": model,
            "optimizer": {k: (v.cpu() if isinstance(v, torch.Tensor) else v)
                          for k, v in trainer.optimizer.state_dict().items()},
            "lr_scheduler": trainer.lr_schedule.state_dict(),
            "random_rng_state": random.getstate(),
            "np_rng_state": np.random.get_state(),
            "torch_rng_state": torch.get_rng_state(),
            "rng_tracker_states": {"dropout_seed_state": F.seed_state().get_state()},
            "buffers": {k: v.cpu().clone() for k, v in _buffers(trainer).items()},
            "plan": trainer.plan,
            "op_names": {i: trainer.op_names[i] for i in trainer.owned_op_indices()},
            "param_specs": {names[s.name]: {"full_shape": s.full_shape, "shard_dim": s.shard_dim, "tp": s.tp,
                                            "tp_rank": s.tp_rank} for s in trainer.store.specs},
        }
        path = os.path.join(d, "model_optim_rng.pt")
        torch.save(sd, path)
    if trainer.world_size > 1:
        torch.distributed.barrier()
    if trainer.rank == 0:
        with open(os.path.join(root, TRACKER), "w") as f:
            f.write(str(it))
    return path


def read_tracker(root: str):
    p = os.path.join(root, TRACKER)
    if not os.path.isfile(p):
        return None
    s = open(p).read().strip()
    return "release" if s == "release" else int(s)


def load_checkpoint(trainer, root: str, load_optim: bool = True, load_rng: bool = True, finetune: bool = False) -> int:
    """Loads the latest checkpoint written under the SAME plan; returns the iteration (0 when none exists)."""
    it = read_tracker(root)
    if it is None:
        return 0
    ps = trainer.pstate
    _, shard = _shard_of(trainer)
    path = os.path.join(checkpoint_dir(root, it, shard, ps.stage, ps.num_stages), "model_optim_rng.pt")
    sd = _load_file(path)
    if sd.get("plan") is not None and sd["plan"]["num_ops_in_each_stage"] != trainer.plan["num_ops_in_each_stage"]:
        raise RuntimeError("checkpoint was written under a different stage split; use load_under_plan()")
    names = _local_names(trainer)
    trainer.store.load_state_dict({k: sd["model"][names[k]] for k in trainer.store.params})
    saved = sd.get("buffers", {})
    if saved:
        # running statistics exist once an op has run: one forward under no_grad creates them, then they are filled
        for op in trainer.stage.raw_ops:
            for owner in (op, getattr(op, "bn_op", None)):
                if owner is not None and hasattr(owner, "_buffers"):
                    owner._buffers(trainer.device)
        for k, v in _buffers(trainer).items():
            if k in saved:
                v.copy_(saved[k].to(v.device))
    if finetune or it == "release":
        trainer.iteration = 0
        return 0
    if load_optim:
        trainer.optimizer.load_state_dict({k: (v.to(trainer.device) if isinstance(v, torch.Tensor) else v)
                                           for k, v in sd["optimizer"].items()})
        trainer.lr_schedule.load_state_dict(sd["lr_scheduler"])
    if load_rng:
        random.setstate(sd["random_rng_state"])
        np.random.set_state(sd["np_rng_state"])
        torch.set_rng_state(sd["torch_rng_state"])
        F.seed_state().set_state(tuple(sd["rng_tracker_states"]["dropout_seed_state"]))
    trainer.iteration = sd["iteration"]
    return trainer.iteration


def merge_tp_shards(root: str, iteration) -> Dict[str, torch.Tensor]:
    """Full (unsharded) model tensors keyed by ``{global op index}.{param}``, from every mp_rank_* directory."""
    tag = "release" if iteration == "release" else "iter_{:07d}".format(iteration)
    base = os.path.join(root, tag)
    pieces: Dict[str, Dict[int, torch.Tensor]] = {}
    meta: Dict[str, dict] = {}
    for sub in sorted(os.listdir(base)):
        sd = _load_file(os.path.join(base, sub, "model_optim_rng.pt"))
        lo = min(sd["op_names"])
        for name, t in sd["model"].items():
            _, _, idx, rest = name.split(".", 3)
            gname = f"{int(idx) + lo}.{rest}"
            spec = sd["param_specs"][name]
            pieces.setdefault(gname, {})[spec["tp_rank"]] = t
            meta[gname] = spec
    full = {}
    for gname, parts in pieces.items():
        spec = meta[gname]
        if spec["shard_dim"] is None or spec["tp"] == 1:
            full[gname] = parts[min(parts)]
        else:
            shards = [parts[r] for r in range(spec["tp"])]
            local_shape = list(spec["full_shape"])
            local_shape[spec["shard_dim"]] //= spec["tp"]
            full[gname] = torch.cat([s.reshape(local_shape) for s in shards], dim=spec["shard_dim"])
    return full


def load_under_plan(trainer, root: str) -> int:
    """Loads model weights from a checkpoint written under ANY plan of the same model (weights only)."""
    it = read_tracker(root)
    if it is None:
        return 0
    full = merge_tp_shards(root, it)
    out = {}
    for s in trainer.store.specs:
        _, idx, rest = s.name.split(".", 2)
        key = f"{idx}.{rest}"
        if key not in full and s.shared_key is not None:   # a tied copy that lived in another op under the old plan
            key = next(k for k in full if k.split(".", 1)[1] == rest)
        t = full[key]
        if s.shard_dim is not None and s.tp > 1:
            t = t.reshape(s.full_shape).chunk(s.tp, dim=s.shard_dim)[s.tp_rank]
        out[s.name] = t.reshape(s.shape)
    trainer.store.load_state_dict(out)
    return it if isinstance(it, int) else 0
