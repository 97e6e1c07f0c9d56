"""Weights shared by ops that live in different pipeline stages (word embeddings used by the embedding op and
by the LM head; T5 also shares them with the decoder embedding, together with the position embeddings).

Every holder initialises its copy from the same seed, so the copies start equal without communication.  After
the backward passes of an iteration the gradients of all copies are summed at the first holder and sent
back, through the relayout engine, which re-splits the vocabulary shards when the holders use different
tensor-parallel degrees (reference: initialize_weights_sharing / synchronize_shared_weights_grads,
runtime/megatron/training.py:227-496).
"""
from __future__ import annotations

from typing import List, Tuple


from ..parallel.relayout import Layout, Side, Transfer

DECLARING_OPS = {
    "word_embeddings": ("encoder-embedding", "decoder-embedding", "gpt-post-process", "t5-post-process",
                        "bert-post-process"),
    "position_embeddings": ("encoder-embedding", "decoder-embedding"),
    # T5 relative-position tables [heads / tp, buckets]: one per stack, used by every layer of the stack
    "enc_relative_attention_bias": ("enc-attention-score",),
    "dec_relative_attention_bias": ("dec-attention-score-1",),
}
LAYOUT = {"word_embeddings": Layout("rep", "split"), "position_embeddings": Layout("rep", "rep"),
          "enc_relative_attention_bias": Layout("rep", "split"), "dec_relative_attention_bias": Layout("rep", "split")}


class TiedWeights:
    def __init__(self, trainer):
        self.t = trainer
        plan, ps = trainer.plan, trainer.pstate
        self.links: List[Tuple[str, Side, Side]] = []   # (shared key, root side, other side)
        for key, op_names in DECLARING_OPS.items():
            if key.endswith("relative_attention_bias") and not getattr(trainer.cfg, "relative_position_bias", False):
                continue
            holders: List[Side] = []
            seen = set()   # (physical stage, tp): one copy per stage and tensor-parallel degree, shared by its ops
            for s, (lo, hi) in enumerate(trainer.stage_bounds):
                phys = s % ps.num_stages
                for i in range(lo, hi):
                    if trainer.op_names[i] in op_names:
                        tp = plan["model_parallel_size_of_each_op"][s][i - lo]
                        if (phys, tp) in seen:
                            continue
                        seen.add((phys, tp))
                        holders.append(Side(ps.stage_start[phys], tp, plan["data_parallel_size_of_each_op"][s][i - lo]))
            for other in holders[1:]:
                self.links.append((key, holders[0], other))

    def duplicate_param_names(self) -> List[str]:
        """Parameters of THIS rank that are non-root copies of a tied weight (counted once in the gradient norm,
        at the root)."""
        out = []
        for key, root, other in self.links:
            if other.contains(self.t.rank):
                name = self.t.store.shared_name(key, other.tp)
                if name is not None:
                    out.append(name)
        return out

    def _grad(self, key: str, tp: int):
        name = self.t.store.shared_name(key, tp)
        return None if name is None else self.t.store.params[name].main_grad

    def sync_grads(self) -> None:
        """Two passes over the links: first every copy's gradient is added at the root, then the total goes back to
        every copy (with three holders -- T5's encoder embedding, decoder embedding and LM head -- a copy must not
        be overwritten before the last contribution has arrived at the root)."""
        rank, dev = self.t.rank, self.t.device
        for phase in ("up", "down"):
            for key, root, other in self.links:
                in_root, in_other = root.contains(rank), other.contains(rank)
                if not (in_root or in_other):
                    continue
                g_root = self._grad(key, root.tp) if in_root else None
                g_other = self._grad(key, other.tp) if in_other else None
                lay = LAYOUT[key]
                ref, side = (g_other, other) if in_other else (g_root, root)
                # global shape of [1, rows, cols] with dim 1 (vocabulary / heads) split over tp
                local = (1,) + tuple(ref.shape)
                gshape = (1, local[1] * (side.tp if lay.col == "split" else 1)) + tuple(local[2:])
                if phase == "up":
                    up = Transfer(rank, other, lay, root, lay, gshape, ref.dtype, dev)
                    got = up.post(g_other.unsqueeze(0).contiguous() if in_other else None)()
                    if in_root:
                        g_root.add_(got.squeeze(0))
                else:
                    down = Transfer(rank, root, lay, other, lay, gshape, ref.dtype, dev)
                    got = down.post(g_root.unsqueeze(0).contiguous() if in_root else None)()
                    if in_other:
                        g_other.copy_(got.squeeze(0))
