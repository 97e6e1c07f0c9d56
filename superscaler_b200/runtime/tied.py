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
    "word_embeddings": ("encoder-embedding", "decoder-embedding", "gpt-post-process", "t5-post-process"),
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
            seen = set()   # physical stages that already hold a copy (one copy per stage, shared by its chunks)
            for s, (lo, hi) in enumerate(trainer.stage_bounds):
                phys = s % ps.num_stages
                if phys in seen:
                    continue
                for i in range(lo, hi):
                    if trainer.op_names[i] in op_names:
                        holders.append(Side(ps.stage_start[phys], plan["model_parallel_size_of_each_op"][s][i - lo],
                                            plan["data_parallel_size_of_each_op"][s][i - lo]))
                        seen.add(phys)
                        break
            for other in holders[1:]:
                self.links.append((key, holders[0], other))

    def duplicate_param_names(self) -> List[str]:
        """Parameters of THIS rank that are non-root copies of a tied weight (counted once in the gradient norm,
        at the root)."""
        out = []
        for key, root, other in self.links:
            if other.contains(self.t.rank):
                name = self.t.store._shared.get(key)
                if name is not None:
                    out.append(name)
        return out

    def _grad(self, key: str):
        name = self.t.store._shared.get(key)
        return None if name is None else self.t.store.params[name].main_grad

    def sync_grads(self) -> None:
        rank, dev = self.t.rank, self.t.device
        for key, root, other in self.links:
            if not (root.contains(rank) or other.contains(rank)):
                continue
            g = self._grad(key)
            lay = LAYOUT[key]
            mine = root if root.contains(rank) else other
            # global shape of [1, rows, cols] with dim 1 (vocabulary) split over tp
            local = (1,) + tuple(g.shape)
            gshape = (1, local[1] * (mine.tp if lay.col == "split" else 1)) + tuple(local[2:])
            up = Transfer(rank, other, lay, root, lay, gshape, g.dtype, dev)
            got = up.post(g.unsqueeze(0).contiguous() if other.contains(rank) else None)()
            if root.contains(rank):
                g.add_(got.squeeze(0))
            down = Transfer(rank, root, lay, other, lay, gshape, g.dtype, dev)
            got = down.post(g.unsqueeze(0).contiguous() if root.contains(rank) else None)()
            if other.contains(rank):
                g.copy_(got.squeeze(0))
