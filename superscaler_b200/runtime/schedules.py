"""Pipeline execution: 1F1B over stages with different GPU counts, plain (PipelineRunner) and interleaved with
several model chunks per stage (InterleavedRunner, program built by interleaved_program).

Schedule (same as the reference's forward_backward_pipelining_without_interleaving,
runtime/megatron/schedules.py:533-646): stage s of P runs min(P - s - 1, M) warm-up forwards, then
alternates one forward and one backward, then drains the remaining backwards.  Send and receive of one
step are issued as ONE batched group call per stage so neighbouring stages never wait on each other's
sends.

Stage-to-stage exchange (reference: _communicate_flexpipe, runtime/megatron/p2p_communication.py:203-337):
the tensors that are live across the boundary (found by the liveness pass over the op list) travel
through the relayout engine, which re-chunks each of them from the producer's (tp, dp) to the consumer's.
Shapes are exchanged once, on the first micro-batch.  There is no host synchronisation besides waiting
for the requests of the current step (the reference also calls torch.cuda.synchronize(),
p2p_communication.py:317-318).
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from ..models.static_info import live_keys_before
from ..parallel.relayout import Layout, Side, Transfer, global_shape

_DTYPES = [torch.bfloat16, torch.float32, torch.int64, torch.float16, torch.uint8, torch.int32]
_META_WORDS = 12  # per key: ndim, dtype, row, col, groups, requires_grad, then up to 6 dims


class Boundary:
    """One side's view of the boundary between stage `up` (producer) and stage `up + 1` (consumer)."""

    def __init__(self, trainer, up: int):
        ps, plan = trainer.pstate, trainer.plan
        self.trainer, self.rank = trainer, ps.rank
        lo_next = trainer.stage_bounds[up + 1][0]
        P = ps.num_stages   # `up` counts virtual stages; virtual stage s runs on physical stage s % P
        self.keys = live_keys_before(trainer.op_names, lo_next)
        tp_a = plan["model_parallel_size_of_each_op"][up][-1]
        dp_a = plan["data_parallel_size_of_each_op"][up][-1]
        tp_b = plan["model_parallel_size_of_each_op"][up + 1][0]
        dp_b = plan["data_parallel_size_of_each_op"][up + 1][0]
        self.src = Side(ps.stage_start[up % P], tp_a, dp_a)
        self.dst = Side(ps.stage_start[(up + 1) % P], tp_b, dp_b)
        self.i_am_src = ps.stage == up % P
        self.meta: Optional[Dict[str, tuple]] = None   # key -> (gshape, dtype, Layout, needs_grad, one_d)
        self.device = trainer.device

    # ---- one-time shape handshake ---------------------------------------------------------------
    def _encode(self, st: Dict[str, Any], sides: Dict[str, tuple]) -> torch.Tensor:
        words = torch.zeros(len(self.keys) * _META_WORDS, dtype=torch.int64)
        for i, k in enumerate(self.keys):
            t = st[k]
            side, lay = sides[k]
            one_d = t.dim() == 1
            shape = global_shape(side, lay, (1,) + tuple(t.shape) if one_d else tuple(t.shape))
            base = i * _META_WORDS
            words[base + 0] = len(shape) | (64 if one_d else 0)
            words[base + 1] = _DTYPES.index(t.dtype)
            words[base + 2] = 1 if lay.row == "split" else 0
            words[base + 3] = 1 if lay.col == "split" else 0
            words[base + 4] = lay.groups
            words[base + 5] = 1 if (t.is_floating_point() and t.requires_grad) else 0
            for j, d in enumerate(shape):
                words[base + 6 + j] = d
        return words

    def _decode(self, words: torch.Tensor) -> None:
        self.meta = {}
        w = words.tolist()
        for i, k in enumerate(self.keys):
            base = i * _META_WORDS
            nd, one_d = w[base] & 63, bool(w[base] & 64)
            lay = Layout("split" if w[base + 2] else "rep", "split" if w[base + 3] else "rep", w[base + 4])
            self.meta[k] = (tuple(w[base + 6: base + 6 + nd]), _DTYPES[w[base + 1]], lay, bool(w[base + 5]), one_d)

    def handshake_send(self, st, sides) -> None:
        words = self._encode(st, sides)
        self._decode(words)
        dev_words = words.to(self.device)
        # source rank i informs the destination ranks i, i + |src|, ...
        mine = [r for j, r in enumerate(range(self.dst.first_rank, self.dst.first_rank + self.dst.size))
                if j % self.src.size == self.rank - self.src.first_rank]
        reqs = [dist.isend(dev_words, r) for r in mine]
        for r in reqs:
            r.wait()

    def handshake_recv(self) -> None:
        words = torch.zeros(len(self.keys) * _META_WORDS, dtype=torch.int64, device=self.device)
        j = self.rank - self.dst.first_rank
        dist.recv(words, self.src.first_rank + j % self.src.size)
        self._decode(words.cpu())

    # ---- transfers ------------------------------------------------------------------------------
    def forward_ops(self, st: Optional[Dict[str, Any]], sides: Optional[Dict[str, tuple]]):
        """P2P ops that move the boundary tensors downstream; returns (ops, assemble() -> (state, sides))."""
        all_ops, parts = [], []
        for k in self.keys:
            gshape, dtype, lay, _, one_d = self.meta[k]
            src_side, src_lay = (sides[k] if self.i_am_src else (self.src, lay))
            t = None
            if self.i_am_src:
                t = st[k].detach()
                t = (t.unsqueeze(0) if one_d else t).contiguous()
            tr = Transfer(self.rank, src_side, src_lay, self.dst, lay, gshape, dtype, self.device)
            ops, asm = tr.prepare(t)
            all_ops += ops
            parts.append((k, asm))

        def assemble():
            out, out_sides = {}, {}
            for k, asm in parts:
                t = asm()
                if t is None:
                    continue
                gshape, dtype, lay, needs_grad, one_d = self.meta[k]
                t = t.squeeze(0) if one_d else t
                if needs_grad and t.is_floating_point():
                    t.requires_grad_(True)
                out[k] = t
                out_sides[k] = (self.dst, lay)
            return out, out_sides

        return all_ops, assemble

    def backward_ops(self, grads: Optional[Dict[str, torch.Tensor]], src_sides: Optional[Dict[str, tuple]]):
        """P2P ops that return the gradients of the boundary tensors upstream; assemble() -> {key: grad}."""
        all_ops, parts = [], []
        for k in self.keys:
            gshape, dtype, lay, needs_grad, one_d = self.meta[k]
            if not needs_grad:
                continue
            up_side, up_lay = (src_sides[k] if self.i_am_src else (self.src, lay))
            g = None
            if not self.i_am_src:
                g = grads[k]
                g = (g.unsqueeze(0) if one_d else g).contiguous()
            tr = Transfer(self.rank, self.dst, lay, up_side, up_lay, gshape, dtype, self.device,
                          sum_row_replicas=True)
            ops, asm = tr.prepare(g)
            all_ops += ops
            parts.append((k, asm, one_d))

        def assemble():
            out = {}
            for k, asm, one_d in parts:
                t = asm()
                if t is not None:
                    out[k] = t.squeeze(0) if one_d else t
            return out

        return all_ops, assemble


def _run_batch(ops):
    reqs = dist.batch_isend_irecv(ops) if ops else []
    for r in reqs:
        r.wait()


class PipelineRunner:
    def __init__(self, trainer):
        self.t = trainer
        ps = trainer.pstate
        self.stage, self.P = ps.stage, ps.num_stages
        self.prev = Boundary(trainer, self.stage - 1) if self.stage > 0 else None
        self.next = Boundary(trainer, self.stage) if self.stage < self.P - 1 else None
        self._next_sides: List[Dict[str, tuple]] = []

    # ---- single steps ---------------------------------------------------------------------------
    def _forward(self, batch, mb: int, received) -> Tuple[Dict[str, Any], Dict[str, Any]]:
        st = self.t.microbatch_inputs(batch, mb)
        st["_meta"] = {}
        inputs = {}
        if received is not None:
            tensors, sides = received
            st.update(tensors)
            st["_meta"].update(sides)
            inputs = tensors
        self.t.stage.forward(st)
        return st, inputs

    def _exchange(self, send_fwd=None, recv_fwd=False, send_bwd=None, recv_bwd=False):
        """One batched group call with every send / receive of this step."""
        ops, got_fwd, got_bwd = [], None, None
        if recv_fwd:
            if self.prev.meta is None:
                self.prev.handshake_recv()
            o, asm_f = self.prev.forward_ops(None, None)
            ops += o
        if send_bwd is not None:
            o, _ = self.prev.backward_ops(send_bwd, None)
            ops += o
        if send_fwd is not None:
            st, sides = send_fwd
            if self.next.meta is None:
                self.next.handshake_send(st, sides)
            o, _ = self.next.forward_ops(st, sides)
            ops += o
        if recv_bwd:
            o, asm_b = self.next.backward_ops(None, recv_bwd)
            ops += o
        _run_batch(ops)
        if recv_fwd:
            got_fwd = asm_f()
        if recv_bwd:
            got_bwd = asm_b()
        return got_fwd, got_bwd

    def _outputs(self, st) -> Tuple[Dict[str, Any], Dict[str, tuple]]:
        keys = self.next.keys
        return {k: st[k] for k in keys}, {k: st["_meta"][k] for k in keys}

    def _backward(self, st, inputs, out_grads, loss_buf) -> Dict[str, torch.Tensor]:
        if self.next is None:
            loss = st["loss"]
            loss.backward()
            loss_buf += loss.detach()
        else:
            outs, gs = [], []
            for k, g in out_grads.items():
                o = st[k]
                if isinstance(o, torch.Tensor) and o.requires_grad:
                    outs.append(o)
                    gs.append(g.to(o.dtype))
            torch.autograd.backward(outs, gs)
        grads = {}
        for k, t in inputs.items():
            if t.is_floating_point() and t.requires_grad:
                grads[k] = t.grad if t.grad is not None else torch.zeros_like(t)
        return grads

    def run_forward_only(self, batch, loss_buf: torch.Tensor) -> torch.Tensor:
        """Evaluation: every micro-batch flows through the stages once, nothing is kept (call under no_grad).
        Uses boundaries of its own, because the tensor descriptions exchanged on first use record whether a
        gradient flows back, which differs between training and evaluation."""
        if not hasattr(self, "_eval_bounds"):
            self._eval_bounds = (Boundary(self.t, self.stage - 1) if self.stage > 0 else None,
                                 Boundary(self.t, self.stage) if self.stage < self.P - 1 else None)
        train_bounds = (self.prev, self.next)
        self.prev, self.next = self._eval_bounds
        try:
            for mb in range(self.t.num_microbatches):
                received = None
                if self.prev is not None:
                    received, _ = self._exchange(recv_fwd=True)
                st, _ = self._forward(batch, mb, received)
                if self.next is None:
                    loss_buf += st["loss"]
                else:
                    self._exchange(send_fwd=self._outputs(st))
        finally:
            self.prev, self.next = train_bounds
        return loss_buf

    # ---- the schedule ---------------------------------------------------------------------------
    def run(self, batch, loss_buf: torch.Tensor) -> torch.Tensor:
        M = self.t.num_microbatches
        warm = min(self.P - self.stage - 1, M)
        steady = M - warm
        first, last = self.prev is None, self.next is None
        pending: List[tuple] = []   # (state, inputs, sides of the sent tensors)
        mb = 0
        received = None
        if not first:
            received, _ = self._exchange(recv_fwd=True)
        for i in range(warm):
            st, inputs = self._forward(batch, mb, received)
            mb += 1
            outs = self._outputs(st)
            pending.append((st, inputs, outs[1]))
            more_fwd = (i + 1 < warm) or steady > 0
            received, _ = self._exchange(send_fwd=outs, recv_fwd=(not first) and more_fwd)
        for i in range(steady):
            st, inputs = self._forward(batch, mb, received)
            mb += 1
            out_grads = None
            if not last:
                outs = self._outputs(st)
                pending.append((st, inputs, outs[1]))
                _, out_grads = self._exchange(send_fwd=outs, recv_bwd=pending[0][2])
            else:
                pending.append((st, inputs, None))
            st_b, in_b, _ = pending.pop(0)
            grads = self._backward(st_b, in_b, out_grads, loss_buf)
            more_fwd = i + 1 < steady
            if not first:
                received, _ = self._exchange(send_bwd=grads, recv_fwd=more_fwd)
        for i in range(warm):
            _, out_grads = self._exchange(recv_bwd=pending[0][2])
            st_b, in_b, _ = pending.pop(0)
            grads = self._backward(st_b, in_b, out_grads, loss_buf)
            if not first:
                self._exchange(send_bwd=grads)
        return loss_buf


# ---- interleaved (virtual-stage) 1F1B ---------------------------------------------------------------

def interleaved_program(P: int, v: int, M: int, p: int, forward_only: bool = False) -> List[tuple]:
    """The ordered program of physical stage `p` for one iteration of interleaved 1F1B with P physical stages,
    v model chunks per stage and M micro-batches (M a multiple of P).

    Entries: ("F", chunk, mb), ("B", chunk, mb) and ("X", [(kind, chunk, mb), ...]) with kind one of send_fwd /
    recv_fwd / send_bwd / recv_bwd; all transfers of one X entry are issued as one batched group call.  Compute
    order (reference: forward_backward_pipelining_with_interleaving, runtime/megatron/schedules.py:232-522):
    micro-batches advance in groups of P through chunk 0, 1, ... v-1; a stage runs
    min(2 (P - p - 1) + (v - 1) P, M v) warm-up forwards (all M v when M == P), then forward / backward pairs, then
    the remaining backwards; backward step k belongs to chunk v - 1 - (k mod P v) // P.  After every compute
    step the stage sends what it produced and receives exactly what its NEXT forward and backward steps consume.
    With forward_only (evaluation) the program is the chain of forward steps alone.
    """
    assert v >= 1 and P >= 1 and M % P == 0, "the number of micro-batches must be a multiple of the stage count"
    T = M * v
    first, last = p == 0, p == P - 1

    def fwd(k):
        return (k % (P * v)) // P, (k // (P * v)) * P + k % P

    def bwd(k):
        c, mb = fwd(k)
        return v - 1 - c, mb

    def recv_fwd(k):   # input of forward step k arrives over the network unless it is the data loader's
        return [("recv_fwd",) + fwd(k)] if k < T and not (first and fwd(k)[0] == 0) else []

    def send_fwd(k):
        return [("send_fwd",) + fwd(k)] if not (last and fwd(k)[0] == v - 1) else []

    def recv_bwd(k):
        return [("recv_bwd",) + bwd(k)] if k < T and not (last and bwd(k)[0] == v - 1) else []

    def send_bwd(k):
        return [("send_bwd",) + bwd(k)] if not (first and bwd(k)[0] == 0) else []

    warm = T if (M == P or forward_only) else min(2 * (P - p - 1) + (v - 1) * P, T)
    rem = T - warm
    prog: List[tuple] = [("X", recv_fwd(0))]
    for k in range(warm):
        prog.append(("F",) + fwd(k))
        ops = send_fwd(k) + recv_fwd(k + 1)
        if k == warm - 1 and not forward_only:
            ops += recv_bwd(0)
        prog.append(("X", ops))
    if forward_only:
        return [e for e in prog if e[0] != "X" or e[1]]
    for k in range(rem):
        fk = k + warm
        prog.append(("F",) + fwd(fk))
        prog.append(("B",) + bwd(k))
        prog.append(("X", send_fwd(fk) + send_bwd(k) + recv_fwd(fk + 1) + recv_bwd(k + 1)))
    for k in range(rem, T):
        prog.append(("B",) + bwd(k))
        prog.append(("X", send_bwd(k) + recv_bwd(k + 1)))
    return [e for e in prog if e[0] != "X" or e[1]]


def simulate_programs(P: int, v: int, M: int, t_fwd: float = 1.0, t_bwd: float = 2.0, forward_only: bool = False):
    """Runs the P programs of interleaved_program against each other on a model of batched point-to-point
    calls: a batch completes when each of its transfers has met the matching transfer of the peer, transfers
    between one pair of stages in one direction match in the order they were posted, and a stage does nothing
    else while a batch is pending.  Returns (finish time, bubble fraction) or raises on a deadlock, on a
    transfer that meets the wrong partner, or on a compute step whose input never arrived.
    """
    progs = [interleaved_program(P, v, M, p, forward_only) for p in range(P)]
    pc = [0] * P
    clock = [0.0] * P
    busy = [0.0] * P
    posted: Dict[tuple, List[tuple]] = {}    # (src stage, dst stage) -> [(payload tag, time posted)] sends
    wanted: Dict[tuple, List[tuple]] = {}    # (src stage, dst stage) -> [(payload tag, time posted)] receives
    have = [set() for _ in range(P)]         # ("act" | "grad", chunk, mb) available at a stage
    done_f = [set() for _ in range(P)]
    pending: List[Optional[list]] = [None] * P   # transfers of the current batch that are still unmatched

    def tag_of(p, kind, c, mb):
        # the payload is named after the virtual boundary it crosses
        s = c * P + p
        if kind == "send_fwd":
            return ("act", s, mb), (p, (p + 1) % P)
        if kind == "recv_fwd":
            return ("act", s - 1, mb), ((p - 1) % P, p)
        if kind == "send_bwd":
            return ("grad", s - 1, mb), (p, (p - 1) % P)
        return ("grad", s, mb), ((p + 1) % P, p)

    progress = True
    while progress:
        progress = False
        for p in range(P):
            while pc[p] < len(progs[p]):
                e = progs[p][pc[p]]
                if e[0] == "F":
                    _, c, mb = e
                    if c * P + p > 0 and ("act", c * P + p - 1, mb) not in have[p]:
                        raise RuntimeError(f"stage {p}: forward of chunk {c} micro-batch {mb} has no input")
                    done_f[p].add((c, mb))
                    clock[p] += t_fwd
                    busy[p] += t_fwd
                elif e[0] == "B":
                    _, c, mb = e
                    if (c, mb) not in done_f[p]:
                        raise RuntimeError(f"stage {p}: backward before forward for chunk {c} micro-batch {mb}")
                    if c * P + p < P * v - 1 and ("grad", c * P + p, mb) not in have[p]:
                        raise RuntimeError(f"stage {p}: backward of chunk {c} micro-batch {mb} has no gradient")
                    clock[p] += t_bwd
                    busy[p] += t_bwd
                else:
                    if pending[p] is None:
                        pending[p] = []
                        for kind, c, mb in e[1]:
                            tag, pair = tag_of(p, kind, c, mb)
                            q = posted if kind.startswith("send") else wanted
                            q.setdefault(pair, []).append((tag, clock[p], p))
                            pending[p].append((kind.startswith("send"), pair, tag))
                    # a transfer is complete when both queues of its pair hold it at matching positions
                    still = []
                    t_done = clock[p]
                    for is_send, pair, tag in pending[p]:
                        mine = posted.get(pair, []) if is_send else wanted.get(pair, [])
                        theirs = wanted.get(pair, []) if is_send else posted.get(pair, [])
                        idx = [i for i, x in enumerate(mine) if x[0] == tag][0]
                        if idx >= len(theirs):
                            still.append((is_send, pair, tag))
                            continue
                        if theirs[idx][0] != tag:
                            raise RuntimeError(f"stage {p}: transfer {tag} met {theirs[idx][0]} on {pair}")
                        t_done = max(t_done, theirs[idx][1])
                        if not is_send:
                            have[p].add(tag)
                    if still:
                        pending[p] = still
                        break
                    pending[p] = None
                    clock[p] = max(clock[p], t_done)
                pc[p] += 1
                progress = True
    if any(pc[p] < len(progs[p]) for p in range(P)):
        raise RuntimeError(f"deadlock at program counters {pc}")
    finish = max(clock)
    return finish, 1.0 - (sum(busy) / P) / finish


class InterleavedRunner:
    """Executes interleaved_program: every physical stage owns v model chunks; chunk c of stage p is virtual
    stage c * P + p and exchanges with virtual stages c * P + p - 1 and c * P + p + 1 (the last stage's chunk c
    feeds the first stage's chunk c + 1).  Activation memory per stage peaks at the warm-up depth of the
    program; the pipeline bubble shrinks by the factor v against plain 1F1B."""

    def __init__(self, trainer):
        self.t = trainer
        ps = trainer.pstate
        self.stage, self.P, self.v = ps.stage, ps.num_stages, trainer.interleave
        self.prev, self.next = self._boundaries()
        self.program = None

    def _boundaries(self):
        total = self.P * self.v
        prev: List[Optional[Boundary]] = []
        nxt: List[Optional[Boundary]] = []
        for c in range(self.v):
            s = c * self.P + self.stage
            prev.append(Boundary(self.t, s - 1) if s > 0 else None)
            nxt.append(Boundary(self.t, s) if s < total - 1 else None)
        return prev, nxt

    def run_forward_only(self, batch, loss_buf: torch.Tensor) -> torch.Tensor:
        """Evaluation pass (call under no_grad); see PipelineRunner.run_forward_only for the separate boundaries."""
        if not hasattr(self, "_eval_bounds"):
            self._eval_bounds = self._boundaries()
            self._eval_program = interleaved_program(self.P, self.v, self.t.num_microbatches, self.stage, True)
        train = (self.prev, self.next, self.program)
        (self.prev, self.next), self.program = self._eval_bounds, self._eval_program
        try:
            return self.run(batch, loss_buf, forward_only=True)
        finally:
            self.prev, self.next, self.program = train

    def _exchange(self, ops_spec, outputs, in_grads, sent_sides):
        """One batched group call.  outputs[(c, mb)] = (tensors, sides) to send downstream, in_grads[(c, mb)] =
        gradients to send upstream, sent_sides[(c, mb)] = layouts of what was sent downstream earlier."""
        ops, fwd_asm, bwd_asm = [], [], []
        for kind, c, mb in ops_spec:
            if kind == "send_fwd":
                st, sides = outputs.pop((c, mb))
                b = self.next[c]
                if b.meta is None:
                    b.handshake_send(st, sides)
                ops += b.forward_ops(st, sides)[0]
            elif kind == "send_bwd":
                ops += self.prev[c].backward_ops(in_grads.pop((c, mb)), None)[0]
            elif kind == "recv_fwd":
                b = self.prev[c]
                if b.meta is None:
                    b.handshake_recv()
                o, asm = b.forward_ops(None, None)
                ops += o
                fwd_asm.append(((c, mb), asm))
            else:
                o, asm = self.next[c].backward_ops(None, sent_sides[(c, mb)])
                ops += o
                bwd_asm.append(((c, mb), asm))
        _run_batch(ops)
        return {k: asm() for k, asm in fwd_asm}, {k: asm() for k, asm in bwd_asm}

    def run(self, batch, loss_buf: torch.Tensor, forward_only: bool = False) -> torch.Tensor:
        t = self.t
        M = t.num_microbatches
        assert M % self.P == 0, "interleaved 1F1B needs a micro-batch count that is a multiple of the stage count"
        if self.program is None:
            self.program = interleaved_program(self.P, self.v, M, self.stage)
        received: Dict[tuple, tuple] = {}      # (chunk, mb) -> (tensors, sides) from upstream
        out_grads: Dict[tuple, dict] = {}      # (chunk, mb) -> gradients from downstream
        outputs: Dict[tuple, tuple] = {}
        in_grads: Dict[tuple, dict] = {}
        sent_sides: Dict[tuple, dict] = {}
        live: Dict[tuple, tuple] = {}          # (chunk, mb) -> (state, inputs) between forward and backward
        for e in self.program:
            if e[0] == "X":
                got_f, got_b = self._exchange(e[1], outputs, in_grads, sent_sides)
                received.update(got_f)
                out_grads.update(got_b)
            elif e[0] == "F":
                _, c, mb = e
                st = t.microbatch_inputs(batch, mb)
                st["_meta"] = {}
                inputs = {}
                if self.prev[c] is not None:
                    tensors, sides = received.pop((c, mb))
                    st.update(tensors)
                    st["_meta"].update(sides)
                    inputs = tensors
                t.stage.forward(st, chunk=c)
                if self.next[c] is not None:
                    keys = self.next[c].keys
                    outputs[(c, mb)] = ({k: st[k] for k in keys}, {k: st["_meta"][k] for k in keys})
                if forward_only:
                    if self.next[c] is None:
                        loss_buf += st["loss"]
                    continue
                live[(c, mb)] = (st, inputs)
                if self.next[c] is not None:
                    sent_sides[(c, mb)] = outputs[(c, mb)][1]
            else:
                _, c, mb = e
                st, inputs = live.pop((c, mb))
                if self.next[c] is None:
                    loss = st["loss"]
                    loss.backward()
                    loss_buf += loss.detach()
                else:
                    outs, gs = [], []
                    for k, g in out_grads.pop((c, mb)).items():
                        o = st[k]
                        if isinstance(o, torch.Tensor) and o.requires_grad:
                            outs.append(o)
                            gs.append(g.to(o.dtype))
                    torch.autograd.backward(outs, gs)
                    sent_sides.pop((c, mb))
                if self.prev[c] is not None:
                    in_grads[(c, mb)] = {k: (x.grad if x.grad is not None else torch.zeros_like(x))
                                         for k, x in inputs.items() if x.is_floating_point() and x.requires_grad}
        return loss_buf


def interleave_plan(plan: dict, v: int, ops_per_virtual_stage: Optional[List[int]] = None) -> dict:
    """Re-cuts a P-stage plan into P * v virtual stages for the interleaved schedule (the role of the reference's
    --interleave-factor, runtime/megatron/arguments.py:778-779, whose plans list the virtual stages explicitly).

    The op list is cut into P * v consecutive slices (equal op counts unless `ops_per_virtual_stage` is given);
    slice s runs on the GPUs of stage s % P and takes that stage's tensor / data parallel degrees, so every stage
    of the input plan must use one (tp, dp) for all of its ops.  Per-op recompute and algorithm choices are kept.
    """
    if v <= 1:
        return plan
    P = len(plan["num_ops_in_each_stage"])
    assert int(plan.get("interleave_factor", 1)) == 1, "plan is already interleaved"
    assert P >= 2, "interleaving needs at least two pipeline stages"
    tps, dps = [], []
    for s in range(P):
        tp, dp = set(plan["model_parallel_size_of_each_op"][s]), set(plan["data_parallel_size_of_each_op"][s])
        assert len(tp) == 1 and len(dp) == 1, f"stage {s} mixes parallel degrees; it cannot be interleaved"
        tps.append(tp.pop())
        dps.append(dp.pop())
    n = sum(plan["num_ops_in_each_stage"])
    total = P * v
    if ops_per_virtual_stage is None:
        per = n // total
        ops_per_virtual_stage = [per + (1 if i < n - per * total else 0) for i in range(total)]
    assert len(ops_per_virtual_stage) == total and sum(ops_per_virtual_stage) == n

    def recut(key):
        flat = [x for stage in plan[key] for x in stage]
        out, at = [], 0
        for c in ops_per_virtual_stage:
            out.append(flat[at:at + c])
            at += c
        return out

    new = dict(plan)
    new.update(
        interleave_factor=v, num_stages=total, num_ops_in_each_stage=list(ops_per_virtual_stage),
        num_gpus=[plan["num_gpus"][s % P] for s in range(total)],
        model_parallel_size_of_each_op=[[tps[s % P]] * c for s, c in enumerate(ops_per_virtual_stage)],
        data_parallel_size_of_each_op=[[dps[s % P]] * c for s, c in enumerate(ops_per_virtual_stage)],
        recompute_ops=recut("recompute_ops"), algo_of_each_op=recut("algo_of_each_op"),
        checkpoint_activations=[any(r) for r in recut("recompute_ops")],
        resharding_stages=[False] * total)
    return new
