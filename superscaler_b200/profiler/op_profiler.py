"""Op profiler: times every op of a model on the target GPUs and writes the database the search reads.

    python -m torch.distributed.run --nproc-per-node <tp> --master-addr 127.0.0.1 \
        -m superscaler_b200.profiler.op_profiler --model-name gpt --model-size 1_3B \
        --prof-tp-size <tp> --prof-mbs-list 1 2 4 8 --prof-algo-list 0 1 --prof-path <db>/

One CSV per (micro-batch, tp, algo): ``{model}_{size}_mbs{m}_tp{t}_algo{a}.csv`` with the reference's columns
``op_name, forward-compute, backward-compute (us), input_size, output_size, weights, activations, fwd_reserved,
bwd_reserved (MB)`` (profiler/op_profiler.py:461-487) plus ``fwd_overlap_comm, bwd_overlap_comm`` (us).

How it measures (reference: profiler/op_profiler.py:283-459 uses wall clock around N calls and one sync):
  * a one-layer instance of the model is built for world size = tp (every op at (tp, dp = 1));
  * ops are visited in order; each op's inputs are the detached outputs of its predecessor;
  * forward and backward are timed separately with CUDA events on the launching stream, after warm-up, as the
    device time per call of `--prof-repeat-times` calls launched back to back (the queue stays full, as in a
    training step); before every call the L2 cache is evicted and the op's direct inputs (forward: its input
    tensors, backward: the incoming gradients) are read once, so that weights and saved activations come from HBM
    while what the previous kernel would just have written is L2-resident as far as it fits -- the state a
    training step leaves; at tp > 1 the op's own collectives are inside the timed region;
  * ops that the runtime executes as one fused kernel when co-located (flash attention; GEMM + epilogue) are
    timed fused: the first member carries the time, the others carry 0, which is what the runtime will see;
  * memory columns come from torch.cuda.memory_allocated / max_memory_allocated deltas around the calls.
"""
from __future__ import annotations

import argparse
import csv
import os
from typing import Dict, List

import torch
import torch.distributed as dist

from ..parallel.state import init_distributed
from ..runtime.stage import run_op
from ..runtime.trainer import Trainer

MB = 1024.0 * 1024.0
HEADER = ["op_name", "forward-compute", "backward-compute", "input_size", "output_size", "weights", "activations",
          "fwd_reserved", "bwd_reserved", "fwd_overlap_comm", "bwd_overlap_comm"]


def one_layer_plan(model: str, shape: dict, mbs: int, tp: int, algo: int, names: List[str], tunable: List[str]) -> dict:
    n = len(names)
    d = dict(shape)
    d.update(model_name=model, global_batch_size=mbs, micro_batch_size=mbs, num_stages=1, num_gpus=[tp],
             checkpoint_activations=[False], resharding_stages=[False], num_ops_in_each_stage=[n],
             model_parallel_size_of_each_op=[[tp] * n], data_parallel_size_of_each_op=[[1] * n],
             recompute_ops=[[0] * n], algo_of_each_op=[[algo if nm in tunable else 0 for nm in names]])
    return d


def _tensor_mb(t) -> float:
    return t.numel() * t.element_size() / MB if isinstance(t, torch.Tensor) else 0.0


_L2_FLUSH = None
_FLUSH_ENABLED = True     # --no-l2-flush times the calls back to back without evicting their operands


def _flush_l2() -> None:
    """Overwrites a buffer twice the size of the L2 cache, so that the next call finds its inputs and weights in
    HBM as it does inside a training step (where thousands of other kernels ran since they were produced)."""
    global _L2_FLUSH
    if not _FLUSH_ENABLED:
        return
    if _L2_FLUSH is None:
        _L2_FLUSH = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    _L2_FLUSH.zero_()


def _evict_then_touch(tensors) -> None:
    """The state a training step leaves in front of an op: weights and saved activations come from HBM (thousands of
    kernels ran since they were last used), but what the PREVIOUS kernel just wrote is still in the 126 MB L2 as far
    as it fits.  So: evict everything, then read the op's direct inputs once (one multi-tensor kernel)."""
    _flush_l2()
    if _FLUSH_ENABLED:
        ts = [t for t in tensors if isinstance(t, torch.Tensor) and t.is_cuda and t.is_floating_point() and t.numel() > 0]
        if ts:
            torch._foreach_norm(ts)


def _span_ms(body, n: int) -> float:
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(n):
        body(i)
    e1.record()
    e1.synchronize()
    return e0.elapsed_time(e1) / n


def _event_ms(fn, repeat: int, warmup: int, inputs=()) -> float:
    """Device time per call of `repeat` calls launched back to back (the queue stays full, as in a training step,
    so the launch latency of short kernels is not charged to the op), each preceded by an L2 eviction and a read of
    the op's direct inputs, whose own time is measured the same way and subtracted."""
    for _ in range(warmup):
        fn()
    flush = _span_ms(lambda i: _evict_then_touch(inputs), repeat)
    both = _span_ms(lambda i: (_evict_then_touch(inputs), fn()), repeat)
    return max(both - flush, 0.0)


def profile_plan(plan: dict, rank: int, world: int, overrides: dict, repeat: int, warmup: int, batch_fn) -> List[list]:
    """Returns the CSV rows (one per op name of the one-layer model)."""
    trainer = Trainer(plan, rank=rank, world_size=world, model_overrides=overrides, lr_warmup_steps=0,
                      fused_comm=True)
    batch = trainer.to_device(batch_fn(plan))
    st = trainer.microbatch_inputs(batch, 0)
    if world > 1:
        st["_meta"] = {}
    rows: Dict[str, list] = {}
    store = trainer.store
    for op in trainer.stage.ops:
        members = getattr(op, "members", [op])
        names = [m.info.name for m in members]
        # tensors that come from the data loader (images, ids, labels) never receive a gradient in training
        snapshot = {k: (v.detach().clone().requires_grad_(v.is_floating_point() and k not in batch)
                        if isinstance(v, torch.Tensor) else v) for k, v in st.items()}

        def fwd(keep=None):
            local = dict(snapshot)
            if "_meta" in local:
                local["_meta"] = dict(local["_meta"])
            run_op(op, local)
            if keep is not None:
                keep.update(local)
            return local

        with torch.no_grad():
            t_fwd = _event_ms(fwd, repeat, warmup, [snapshot.get(k) for k in op.reads])
        # backward: fresh forward (untimed) + timed backward of all floating outputs
        def fwd_bwd_setup():
            out = fwd()
            outs = [out[k] for k in op.writes if isinstance(out.get(k), torch.Tensor) and out[k].requires_grad]
            return out, outs

        def timed_bwd(n):
            """n backward passes launched back to back over n separately prepared forward graphs (L2 flushed
            before each, flush time subtracted)."""
            prepared = [fwd_bwd_setup() for _ in range(n)]
            if not prepared[0][1]:
                return 0.0
            grads = [[torch.ones_like(o) if o.dim() == 0 else torch.randn_like(o) for o in outs] for _, outs in prepared]
            flush = _span_ms(lambda i: _evict_then_touch(grads[i]), n)

            def one(i):
                _evict_then_touch(grads[i])     # the incoming gradients were just written; saved activations are cold
                torch.autograd.backward(prepared[i][1], grads[i])

            return max(_span_ms(one, n) - flush, 0.0)

        timed_bwd(min(warmup, 2))
        t_bwd = timed_bwd(repeat)
        store.zero_grad()
        # memory
        torch.cuda.synchronize()
        torch.cuda.reset_peak_memory_stats()
        m0 = torch.cuda.memory_allocated()
        out, outs = fwd_bwd_setup()
        torch.cuda.synchronize()
        m1 = torch.cuda.memory_allocated()
        peak_f = torch.cuda.max_memory_allocated()
        out_mb = sum(_tensor_mb(out.get(k)) for k in op.writes if k != "loss")
        in_mb = sum(_tensor_mb(snapshot.get(k)) for k in op.reads if k not in ("ids", "dec_ids", "labels", "loss_mask"))
        act_mb = max(0.0, (m1 - m0) / MB)
        res_f = max(0.0, (peak_f - m1) / MB)
        torch.cuda.reset_peak_memory_stats()
        if outs:
            torch.autograd.backward(outs, [torch.ones_like(o) if o.dim() == 0 else torch.randn_like(o) for o in outs])
        torch.cuda.synchronize()
        res_b = max(0.0, (torch.cuda.max_memory_allocated() - m1) / MB)
        store.zero_grad()
        w_mb = 0.0
        for m in members:
            for pname in m._names.values():
                p = store.params[pname]
                w_mb += p.numel() * 2 / MB  # bf16 model copy; the cost model multiplies for grads / master / Adam
        # advance the real state
        with torch.no_grad():
            adv = fwd()
        st = {k: v for k, v in adv.items()}
        # the fused group is charged to its first member; sizes follow the x tensor seen at each member boundary
        for i, nm in enumerate(names):
            first = i == 0
            rows[nm] = [nm, f"{(t_fwd * 1000 if first else 0):.3f}", f"{(t_bwd * 1000 if first else 0):.3f}",
                        f"{in_mb:.3f}", f"{out_mb:.3f}", f"{(w_mb if first else 0):.3f}",
                        f"{(act_mb if first else 0):.3f}", f"{(res_f if first else 0):.3f}",
                        f"{(res_b if first else 0):.3f}", "0.000", "0.000"]
        del out, outs, adv, snapshot
    return [rows[n] for n in trainer.op_names]


# ---- model tables ---------------------------------------------------------------------------------
def model_table(model: str, size: str):
    """(plan shape keys, Trainer overrides, op names of a one-layer instance, tunable ops, batch function)."""
    from ..data import synthetic as syn
    from ..search import config as sc
    from ..search import opinfo
    if model == "gpt":
        from ..models.gpt import gpt_op_names
        L, seq, hidden, ffn, heads, kv, vocab, _ = sc.B200_GPT_SIZES.get(size, sc.GPT_SIZES[size])
        shape = dict(model_size=size, num_layers=1, seq_length=seq, max_position_embeddings=seq,
                     num_attention_heads=heads, hidden_size=hidden, kv_channels=kv, ffn_hidden_size=ffn,
                     vocab_size=vocab)
        return (shape, {}, gpt_op_names(1), opinfo.GPT_TUNABLE,
                lambda plan: syn.gpt_batch(plan["global_batch_size"], seq, vocab, seed=1))
    if model == "t5":
        from ..models.t5 import t5_op_names
        L, es, ds, hidden, ffn, heads, kv, vocab, _ = sc.B200_T5_SIZES.get(size, sc.T5_SIZES[size])
        shape = dict(model_size=size, num_layers=1, encoder_seq_length=es, decoder_seq_length=ds,
                     max_position_embeddings=es, num_attention_heads=heads, kv_channels=kv, hidden_size=hidden,
                     ffn_hidden_size=ffn, vocab_size=vocab)
        if size in sc.B200_T5_SIZES:   # the B200 definition: ReLU feed-forward, relative-position buckets (as the search writes it)
            shape.update(activation="relu", relative_position_bias=True, relative_attention_num_buckets=32)
        return (shape, {}, t5_op_names(1), opinfo.T5_TUNABLE,
                lambda plan: syn.t5_batch(plan["global_batch_size"], es, ds, vocab, seed=1))
    if model == "bert":
        from ..models.bert import bert_op_names
        L, seq, hidden, ffn, heads, kv, vocab, _ = sc.BERT_SIZES[size]
        shape = dict(model_size=size, num_layers=1, seq_length=seq, max_position_embeddings=seq,
                     num_attention_heads=heads, hidden_size=hidden, kv_channels=kv, ffn_hidden_size=ffn, vocab_size=vocab)
        return (shape, {}, bert_op_names(1), opinfo.GPT_TUNABLE,
                lambda plan: syn.bert_batch(plan["global_batch_size"], seq, vocab, seed=1))
    if model == "vit":
        from ..models.vit import vit_op_names
        L, image, patch, hidden, ffn, heads, kv, classes, _ = sc.VIT_SIZES[size]
        shape = dict(model_size=size, num_layers=1, image_size=image, patch_dim=patch, num_classes=classes,
                     num_attention_heads=heads, hidden_size=hidden, kv_channels=kv, ffn_hidden_size=ffn)
        return (shape, {}, vit_op_names(1), [op for op in opinfo.GPT_TUNABLE if op != "encoder-embedding"],
                lambda plan: syn.resnet_batch(plan["global_batch_size"], image, classes, seed=1))
    if model == "resnet":
        from ..models.resnet import ResNetConfig, resnet_op_names
        blocks, cin, wf, _ = sc.RESNET_SIZES[size]
        shape = dict(model_size=size, num_layers=list(blocks), in_channels=cin, width_factor=wf)
        names = resnet_op_names(ResNetConfig(blocks=tuple(blocks), in_channels=cin, width_factor=wf))
        tun = [n for n in names if "conv" in n or "downsample" in n]
        return (shape, {}, names, tun, lambda plan: syn.resnet_batch(plan["global_batch_size"], 224, 1000, seed=1))
    raise ValueError(model)


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model-name", required=True)
    ap.add_argument("--model-size", required=True)
    ap.add_argument("--prof-tp-size", type=int, default=None, help="default: WORLD_SIZE")
    ap.add_argument("--prof-mbs-list", nargs="+", type=int, default=None)
    ap.add_argument("--prof-algo-list", nargs="+", type=int, default=None)
    ap.add_argument("--prof-path", required=True)
    ap.add_argument("--prof-repeat-times", type=int, default=10)
    ap.add_argument("--prof-warmup-times", type=int, default=3)
    ap.add_argument("--no-l2-flush", action="store_true",
                    help="do not evict the L2 cache before every timed call (operands of small ops then stay "
                         "cached between the repeats)")
    args = ap.parse_args(argv)
    global _FLUSH_ENABLED
    _FLUSH_ENABLED = not args.no_l2_flush
    rank, world, _ = init_distributed()
    tp = args.prof_tp_size or world
    assert tp == world, "launch exactly tp ranks"
    os.makedirs(args.prof_path, exist_ok=True)
    shape, overrides, names, tunable, batch_fn = model_table(args.model_name, args.model_size)
    mbs_list = args.prof_mbs_list or ([16, 32, 48, 64] if args.model_name == "resnet" else [1, 2, 4, 8])
    algos = args.prof_algo_list or ([0] if args.model_name == "t5" else [0, 1])
    for mbs in mbs_list:
        for algo in algos:
            if algo == 1 and tp == 1:
                pass  # at tp = 1 both algorithms run the same kernels; still measured so the table is complete
            plan = one_layer_plan(args.model_name, shape, mbs, tp, algo, names, tunable)
            try:
                rows = profile_plan(plan, rank, world, overrides, args.prof_repeat_times, args.prof_warmup_times,
                                    batch_fn)
            except torch.cuda.OutOfMemoryError:
                rows = [[n, "10000000", "10000000", "0", "0", "0", "10000000", "0", "0", "0", "0"] for n in names]
                torch.cuda.empty_cache()
            if rank == 0:
                path = f"{args.prof_path}{args.model_name}_{args.model_size}_mbs{mbs}_tp{tp}_algo{algo}.csv"
                with open(path, "w", newline="") as f:
                    w = csv.writer(f)
                    w.writerow(HEADER)
                    w.writerows(rows)
                print(f"wrote {path}", flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
