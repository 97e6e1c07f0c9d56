"""Training driver: builds this rank's stage from a plan JSON and runs iterations.

Public API (what a user calls):

    trainer = Trainer.from_plan("plan.json", model_overrides={...})
    for batch in loader:                      # pinned host tensors, one global batch
        stats = trainer.train_step(batch)     # -> {"loss_tensor": device scalar, "lr": ..., "iteration": ...}
        loss = trainer.loss_value(stats)      # host float (synchronises; averaged over the data-parallel ranks)
    trainer.evaluate(batches)                 # mean loss / perplexity without touching gradients
    trainer.logits(ids)                       # inference forward of a single-stage GPT plan

Counterpart of the reference's pretrain / train_step (runtime/megatron/training.py:83-168,656-752) with
these differences: gradients accumulate in fp32 directly from the wgrad kernels; the optimizer step,
clipping and the inf/nan skip run on the device without a host sync; timing uses CUDA events.
"""
from __future__ import annotations

import json
from typing import Any, Dict, List, Optional

import torch
import torch.distributed as dist

from ..models.base import Env, OpInfo
from ..ops import functional as F
from ..parallel.state import ParallelState
from .lr import LRSchedule
from .optimizer import StageOptimizer
from .params import ParamStore
from .stage import Stage


def _model_factory(model_name: str):
    if model_name == "gpt":
        from ..models import gpt as m
        from ..models.fused import fuse_ops
        return (m.gpt_config_from_plan, lambda c: m.gpt_op_names(c.num_layers),
                lambda i, c: m.gpt_layer_of(i, c.num_layers), m.build_gpt_op, fuse_ops)
    if model_name == "t5":
        from ..models import t5 as m
        from ..models.fused import fuse_ops
        return (m.t5_config_from_plan, lambda c: m.t5_op_names(c.num_layers),
                lambda i, c: m.t5_layer_of(i, c.num_layers), m.build_t5_op, fuse_ops)
    if model_name == "bert":
        from ..models import bert as m
        from ..models.fused import fuse_ops
        return (m.bert_config_from_plan, lambda c: m.bert_op_names(c.num_layers),
                lambda i, c: m.bert_layer_of(i, c.num_layers), m.build_bert_op, fuse_ops)
    if model_name == "ict":
        from ..models import ict as m
        from ..models.fused import fuse_ops
        return (m.ict_config_from_plan, lambda c: m.ict_op_names(c.num_layers),
                lambda i, c: m.ict_layer_of(i, c.num_layers), m.build_ict_op, fuse_ops)
    if model_name == "vit":
        from ..models import vit as m
        from ..models.fused import fuse_ops
        return (m.vit_config_from_plan, lambda c: m.vit_op_names(c.num_layers),
                lambda i, c: m.vit_layer_of(i, c.num_layers), m.build_vit_op, fuse_ops)
    if model_name == "resnet":
        from ..models import resnet as m
        return (m.resnet_config_from_plan, m.resnet_op_names, m.resnet_layer_of, m.build_resnet_op,
                m.fuse_resnet_ops)
    raise ValueError(f"unknown model {model_name}")


# ops that keep their activations whatever the plan says: the embeddings and the loss ops (the search never marks
# them either, reference: search/model_ops_info.py:76-90)
_NEVER_RECOMPUTED = ("encoder-embedding", "decoder-embedding", "gpt-post-process", "t5-post-process",
                     "bert-post-process", "ict-post-process", "vit-embedding", "vit-post-process", "fc")


def _validate_plan(plan: dict) -> None:
    """Shape checks of a plan JSON with messages that name the offending stage (a wrong plan otherwise fails deep
    inside group creation or a kernel launch)."""
    counts = plan["num_ops_in_each_stage"]
    keys = ("model_parallel_size_of_each_op", "data_parallel_size_of_each_op", "algo_of_each_op", "recompute_ops")
    for k in keys:
        if len(plan[k]) != len(counts):
            raise ValueError(f"plan[{k!r}] lists {len(plan[k])} stages, num_ops_in_each_stage lists {len(counts)}")
    if len(plan["num_gpus"]) != len(counts):
        raise ValueError(f"num_gpus lists {len(plan['num_gpus'])} stages, num_ops_in_each_stage lists {len(counts)}")
    for s, n in enumerate(counts):
        for k in keys:
            if len(plan[k][s]) != n:
                raise ValueError(f"stage {s}: {k} has {len(plan[k][s])} entries for {n} ops")
        g = plan["num_gpus"][s]
        for i, (tp, dp) in enumerate(zip(plan["model_parallel_size_of_each_op"][s],
                                         plan["data_parallel_size_of_each_op"][s])):
            if tp * dp != g:
                raise ValueError(f"stage {s} op {i}: tp {tp} x dp {dp} does not equal the stage's {g} GPUs")
            if plan["micro_batch_size"] % dp:
                raise ValueError(f"stage {s} op {i}: dp {dp} does not divide the micro batch {plan['micro_batch_size']}")
        if plan.get("model_name") == "t5" and len(set(plan["data_parallel_size_of_each_op"][s])) > 1:
            # as in the reference (search/aceso_utils.py:523-526): the decoder's tokens enter in the middle of a
            # stage, cut for the stage's first op
            raise ValueError(f"stage {s}: a T5 stage keeps one tensor / data parallel layout for all its ops")


class Trainer:
    def __init__(self, plan: dict, *, rank: int = 0, world_size: int = 1, device=None, seed: int = 1234,
                 model_overrides: Optional[dict] = None, lr: float = 1.5e-4, min_lr: float = 1e-5,
                 weight_decay: float = 0.01, clip_grad: float = 1.0, lr_decay_steps: int = 320000,
                 lr_warmup_steps: int = 3200, lr_style: str = "cosine", optimizer: str = "adam",
                 fuse: bool = True, fused_comm: bool = True, training: bool = True, shard_optimizer: bool = True,
                 distribute_checkpointed_activations: bool = False, adam_betas=(0.9, 0.999), adam_eps: float = 1e-8,
                 sgd_momentum: float = 0.9):
        self.plan = plan
        self.rank, self.world_size = rank, world_size
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        self.device = torch.device(device)
        self.model_name = plan["model_name"]
        cfg_fn, names_fn, layer_fn, build_fn, fuse_fn = _model_factory(self.model_name)
        self.cfg = cfg_fn(plan, **(model_overrides or {}))
        self.global_bs = plan["global_batch_size"]
        self.micro_bs = plan["micro_batch_size"]
        if self.global_bs % self.micro_bs:
            raise ValueError(f"micro batch size {self.micro_bs} does not divide the global batch {self.global_bs}")
        self.num_microbatches = self.global_bs // self.micro_bs
        _validate_plan(plan)
        names = names_fn(self.cfg)
        counts = plan["num_ops_in_each_stage"]
        assert sum(counts) == len(names), f"plan covers {sum(counts)} ops, model has {len(names)}"
        # Interleaving: the plan lists P * v virtual stages in model order; virtual stage s runs on the GPUs of
        # physical stage s % P, so every physical stage owns v model chunks (reference: --interleave-factor,
        # runtime/megatron/arguments.py:778, and get_op_start_index, runtime/megatron/mpu/initialize.py:451-461).
        self.interleave = v = int(plan.get("interleave_factor", 1))
        assert len(counts) % v == 0, "interleave_factor must divide the number of (virtual) stages"
        P = len(counts) // v
        gpus = list(plan["num_gpus"])
        assert len(gpus) == len(counts) and all(gpus[s] == gpus[s % P] for s in range(len(counts))), \
            "every chunk of a physical stage must use that stage's GPUs"
        self.pstate = ParallelState(gpus[:P], rank, world_size)
        self.op_names = names
        self.stage_bounds = [(sum(counts[:i]), sum(counts[:i + 1])) for i in range(len(counts))]
        # every process group any op needs, created in the same order on all ranks
        if world_size > 1:
            pairs = [[] for _ in range(P)]
            for s in range(len(counts)):
                pairs[s % P] += list(zip(plan["model_parallel_size_of_each_op"][s],
                                         plan["data_parallel_size_of_each_op"][s]))
            self.pstate.ensure_groups(self.pstate.all_op_groups(pairs))
        self.virtual_stages = [c * P + self.pstate.stage for c in range(v)]
        chunks = []
        for s in self.virtual_stages:
            lo, hi = self.stage_bounds[s]
            chunks.append([OpInfo(name=names[i], index=i, layer=layer_fn(i, self.cfg),
                                  tp=plan["model_parallel_size_of_each_op"][s][i - lo],
                                  dp=plan["data_parallel_size_of_each_op"][s][i - lo],
                                  algo=plan["algo_of_each_op"][s][i - lo],
                                  recompute=0 if names[i] in _NEVER_RECOMPUTED else plan["recompute_ops"][s][i - lo])
                           for i in range(lo, hi)])
        self.infos = [i for c in chunks for i in c]
        F.manual_seed(seed + 100 * self.pstate.stage)
        self.store = ParamStore(self.device, base_seed=seed)
        # peer-mapped gradient / weight buffers need every rank of the data-parallel group on ONE node (NVLink);
        # a job that spans nodes reduces its gradients with NCCL
        pure_dp = (len(counts) == 1 and world_size > 1 and self.device.type == "cuda" and
                   all(t == 1 for t in plan["model_parallel_size_of_each_op"][0]) and
                   all(d == world_size for d in plan["data_parallel_size_of_each_op"][0]) and
                   self.pstate.same_node(range(world_size)))
        if fused_comm and pure_dp:
            from ..parallel.symm import SymmetricBuffer
            self.store.grad_allocator = lambda n: SymmetricBuffer(n, torch.float32, None, self.device)
            if shard_optimizer:
                # the bf16 model copy is peer-mapped too: each rank updates one slice of the weights and writes the
                # result into every rank's copy
                self.store.model16_allocator = lambda n: SymmetricBuffer(n, torch.bfloat16, None, self.device)
        self.env = Env(cfg=self.cfg, pstate=self.pstate, store=self.store, micro_bs=self.micro_bs,
                       fused_comm=fused_comm, distribute_saved_activations=distribute_checkpointed_activations)
        self.env.training = training
        self.stage = Stage(chunks, self.env, build_fn, fuse_fn if fuse else None)
        self._tied = None
        if world_size > 1:
            # copies of a tied weight in other pipeline stages, or in ops of this stage with another tensor-parallel
            # degree, are kept equal by summing their gradients every step
            from .tied import TiedWeights
            tied = TiedWeights(self)
            self._tied = tied if tied.links else None
        self.optimizer = StageOptimizer(self.store, self.pstate, lr=lr, weight_decay=weight_decay, clip_grad=clip_grad,
                                        kind=optimizer, betas=tuple(adam_betas), eps=adam_eps, momentum=sgd_momentum,
                                        norm_exclude=self._tied.duplicate_param_names() if self._tied else ())
        self.lr_schedule = LRSchedule(lr, min_lr, lr_warmup_steps, lr_decay_steps, lr_style)
        self.iteration = 0
        self.pipeline = None
        if self.pstate.num_stages > 1:
            from .schedules import InterleavedRunner, PipelineRunner
            self.pipeline = InterleavedRunner(self) if v > 1 else PipelineRunner(self)
        self._loss_buf = torch.zeros(1, dtype=torch.float32, device=self.device)
        self.timers: Dict[str, float] = {}

    @classmethod
    def from_plan(cls, path: str, **kw) -> "Trainer":
        with open(path) as f:
            plan = json.load(f)
        return cls(plan, **kw)

    # ---- batches ----------------------------------------------------------------------------
    def first_op_dp(self):
        return self.infos[0].dp

    def local_rows(self, info: OpInfo, total: int) -> slice:
        """Rows of the stage-aggregate micro-batch that belong to this rank for an op with degree dp."""
        pl = self.pstate.placement(info.tp, info.dp)
        per = total // info.dp
        return slice(pl.dp_rank * per, (pl.dp_rank + 1) * per)

    def microbatch_inputs(self, batch: Dict[str, torch.Tensor], mb: int) -> Dict[str, Any]:
        """Device-side slice of micro-batch `mb` for this rank (first stage: inputs, last stage: labels)."""
        st: Dict[str, Any] = {}
        lo = mb * self.micro_bs
        first, last = self.infos[0], self.infos[-1]
        for k, v in batch.items():
            info = last if k in ("labels", "loss_mask", "nsp") else first
            rows = self.local_rows(info, self.micro_bs)
            st[k] = v[lo + rows.start: lo + rows.stop]
        if "enc_lens" in batch:
            # the lengths of the WHOLE micro-batch: an attention op whose data-parallel degree differs from the
            # stage's first op (a plan that changes layouts inside a stage) cuts its own rows out of them
            st["enc_lens_all"] = batch["enc_lens"][lo: lo + self.micro_bs]
        st["loss_scale"] = 1.0 / self.num_microbatches
        return st

    def to_device(self, batch: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        return {k: (v.to(self.device, non_blocking=True) if isinstance(v, torch.Tensor) else v)
                for k, v in batch.items()}

    # ---- one iteration ----------------------------------------------------------------------
    def forward_backward(self, batch: Dict[str, torch.Tensor]) -> torch.Tensor:
        """Runs all micro-batches; returns the summed (already averaged-per-micro-batch) loss on device."""
        self._loss_buf.zero_()
        if self.pipeline is not None:
            return self.pipeline.run(batch, self._loss_buf)
        for mb in range(self.num_microbatches):
            st = self.microbatch_inputs(batch, mb)
            if self.world_size > 1:
                st["_meta"] = {}
            self.stage.forward(st)
            loss = st["loss"]
            loss.backward()
            self._loss_buf += loss.detach()
        return self._loss_buf

    def _fold_autograd_grads(self) -> None:
        """Gradients that reached a parameter through plain autograd (not a fused wgrad kernel)."""
        for p in self.store.params.values():
            if p.grad is not None:
                p.main_grad.add_(p.grad.to(torch.float32))
                p.grad = None

    def train_step(self, batch: Dict[str, torch.Tensor]) -> Dict[str, Any]:
        """One optimizer step on one global batch.  `batch` may live in pinned host memory."""
        batch = self.to_device(batch)
        loss = self.forward_backward(batch)
        self._fold_autograd_grads()
        self.optimizer.reduce_gradients()
        if self._tied is not None:
            self._tied.sync_grads()
        lr = self.lr_schedule.get_lr()          # the reference steps its scheduler after the update
        self.optimizer.step(lr=lr)              # (runtime/megatron/training.py:735-742): update k uses lr(k)
        self.lr_schedule.step()
        self.iteration += 1
        return {"loss_tensor": loss, "lr": lr, "iteration": self.iteration}

    def _read_device_status(self) -> int:
        """The kernels' status word of this device (0 = every bounded wait completed).  Synchronises."""
        from ..ops import native
        if self.device.type != "cuda" or not native.available():
            return 0
        code = native.check_status()
        if code:
            native.ext().status().zero_()
        return code

    def check_device_status(self) -> None:
        """Raises DeviceStatusError when a kernel of this rank gave up a bounded wait since the last check: the data
        of that call (reduced gradients, a fused GEMM's output) is undefined, so the weights must not be trusted or
        saved.  Called where the host synchronises anyway: `loss_value` and `save_checkpoint`.  With a
        `health_monitor` attached the failure is published to the other ranks before the exception leaves."""
        code = self._read_device_status()
        from ..parallel.guards import REGISTRY
        damaged = REGISTRY.check() if REGISTRY.buffers else []
        if code == 0 and not damaged:
            return
        from .health import DeviceStatusError, device_status_message
        if damaged:      # guard words around a peer-written buffer were overwritten (SSB_CANARIES=1)
            err = DeviceStatusError(code, f"iteration {self.iteration}: " + "; ".join(damaged) + "; memory next to a "
                                    "symmetric buffer was written, later weights are not to be saved")
        else:
            err = DeviceStatusError(code, f"iteration {self.iteration}: {device_status_message(code)}; the results of "
                                          "that kernel are undefined, later weights are not to be saved")
        monitor = getattr(self, "health_monitor", None)
        if monitor is not None:
            monitor.publish_failure(f"DeviceStatusError: {err}")
        raise err

    def loss_value(self, stats: Dict[str, Any]) -> float:
        """Host read of the iteration loss (synchronises); averaged over the last stage's DP group.  Also reads
        the kernels' status word and raises if a bounded wait ran out."""
        return float(self._last_stage_mean(stats["loss_tensor"]).item())

    def _last_stage_mean(self, values: torch.Tensor) -> torch.Tensor:
        """Per-iteration values the last stage's ranks hold (each its data-parallel share's mean; tensor-parallel
        replicas repeat it), averaged and made known to every rank.  Checks the kernels' status word first."""
        self.check_device_status()
        t = values.clone()
        if self.world_size > 1:
            last = len(self.stage_bounds) - 1
            if not self.pstate.is_last_stage():
                t.zero_()
            dist.all_reduce(t)
            t /= self.plan["num_gpus"][last]
        return t

    @torch.no_grad()
    def embed(self, batch: Dict[str, torch.Tensor]) -> torch.Tensor:
        """Inference forward of a ONE-stage plan on one rank's rows: the last op's `logits` entry for the given inputs
        (an inverse-cloze plan: one embedding per sequence; BERT: vocabulary logits; ViT / Wide-ResNet: class scores).  `batch` holds the model's input
        keys (ids, types, enc_lens, images ...) and no labels.  Dropout is off."""
        assert len(self.stage_bounds) == 1 and self.world_size == 1, "embed() runs one-stage plans on one rank"
        was = self.env.training
        self.env.training = False
        try:
            st: Dict[str, Any] = {k: (v.to(self.device) if isinstance(v, torch.Tensor) else v) for k, v in batch.items()
                                  if k not in ("labels", "loss_mask", "nsp")}
            self.stage.forward(st)
            return st["logits"]
        finally:
            self.env.training = was

    @torch.no_grad()
    def logits(self, ids: torch.Tensor) -> torch.Tensor:
        """Inference forward of a GPT plan (one stage or a pipeline, any per-op tensor / data parallel layout; not
        interleaved): token ids [b, seq_length] -> logits [b, seq_length, padded vocabulary] on every rank.  Every
        rank passes the same ids.  Rows are split over the data-parallel ranks like a micro-batch (b is padded to a
        multiple of the data-parallel degrees and cut again), the stages hand the activations on once, and the last
        stage shares the logits with the others.  Dropout is off; nothing is kept for a backward pass."""
        import math
        from ..parallel import mappings as M
        from .schedules import Boundary, _run_batch
        assert self.interleave == 1, "logits() does not run interleaved plans; reload the checkpoint under a plain one"
        ps = self.pstate
        b, s = ids.shape
        mult = math.lcm(*(d for stage in self.plan["data_parallel_size_of_each_op"] for d in stage))
        total = -(-b // mult) * mult
        if total != b:
            ids = torch.cat([ids, ids.new_zeros(total - b, s)])
        prev = Boundary(self, ps.stage - 1) if ps.stage > 0 else None
        nxt = Boundary(self, ps.stage) if ps.stage < ps.num_stages - 1 else None
        was = self.env.training
        self.env.training = False
        out = None
        try:
            st: Dict[str, Any] = {}
            if self.world_size > 1:
                st["_meta"] = {}
            if prev is None:
                st["ids"] = ids[self.local_rows(self.infos[0], total)].to(self.device)
            else:
                prev.handshake_recv()
                ops, assemble = prev.forward_ops(None, None)
                _run_batch(ops)
                tensors, sides = assemble()
                st.update(tensors)
                st["_meta"].update(sides)
            self.stage.forward(st)
            if nxt is not None:
                sent = {k: st[k] for k in nxt.keys}
                sides = {k: st["_meta"][k] for k in nxt.keys}
                nxt.handshake_send(sent, sides)
                _run_batch(nxt.forward_ops(sent, sides)[0])
            else:
                last = self.infos[-1]
                pl = ps.placement(last.tp, last.dp)
                out = M.gather_from_group(st["logits"], 0, ps.group(pl.dp_ranks)).contiguous()
        finally:
            self.env.training = was
        if ps.num_stages > 1:
            src = ps.stage_start[-1]
            head = [(tuple(out.shape), out.dtype) if ps.rank == src else None]
            dist.broadcast_object_list(head, src)
            if out is None:
                out = torch.empty(head[0][0], dtype=head[0][1], device=self.device)
            dist.broadcast(out, src)
        return out.view(total, s, -1)[:b]

    @torch.no_grad()
    def evaluate(self, batches) -> Dict[str, float]:
        """Mean loss over an iterable of global batches without touching gradients or optimizer state
        (reference: evaluate / evaluate_and_print_results, runtime/megatron/training.py:1021-1098)."""
        was = self.env.training
        self.env.training = False
        # the classifiers' heads report [loss, top-1 accuracy] in evaluation; both take the same route to the host
        classifier = self.model_name in ("resnet", "vit")
        buf = torch.zeros(2 if classifier else 1, dtype=torch.float32, device=self.device)
        total, n = torch.zeros(buf.numel(), dtype=torch.float64), 0
        try:
            for batch in batches:
                batch = self.to_device(batch)
                buf.zero_()
                if self.pipeline is not None:
                    self.pipeline.run_forward_only(batch, buf)
                else:
                    for mb in range(self.num_microbatches):
                        st = self.microbatch_inputs(batch, mb)
                        if self.world_size > 1:
                            st["_meta"] = {}
                        self.stage.forward(st)
                        buf += st["loss"]
                total += self._last_stage_mean(buf).double().cpu()
                n += 1
        finally:
            self.env.training = was
        mean = float(total[0]) / max(n, 1)
        out = {"lm loss": mean, "lm loss ppl": float(torch.exp(torch.tensor(min(mean, 20.0))))}
        if classifier:
            out = {"lm loss": mean, "accuracy": float(total[1]) / max(n, 1)}
        return out

    def owned_op_indices(self) -> List[int]:
        """Global indices of the ops this rank's physical stage runs (all of its model chunks)."""
        return [i.index for i in self.infos]

    def num_parameters(self) -> int:
        return sum(p.numel() for p in self.store.params.values())
