"""Interleaved (virtual-stage) 1F1B: the per-stage programs are checked against each other on a model of batched
point-to-point calls (matching, input availability, absence of deadlock, pipeline bubble), and multi-rank runs on
CPU (gloo) must reproduce the losses of the single-process run -- the reference's interleaved schedule is
runtime/megatron/schedules.py:232-522."""
import pytest
import torch

from superscaler_b200.data.synthetic import gpt_batch
from superscaler_b200.runtime import checkpointing
from superscaler_b200.runtime.schedules import interleave_plan, interleaved_program, simulate_programs
from superscaler_b200.runtime.trainer import Trainer

from dist_utils import run_ranks
from helpers import tiny_gpt_plan

NODROP = dict(hidden_dropout=0.0, attention_dropout=0.0, max_tp=2)
KW = dict(layers=4, seq=32, hidden=64, heads=2, head_dim=32, vocab=256, global_bs=12, micro_bs=2)


@pytest.mark.parametrize("P", [2, 3, 4, 8])
@pytest.mark.parametrize("v", [1, 2, 3, 4])
def test_programs_match_and_reach_the_ideal_bubble(P, v):
    for M in (P, 2 * P, 4 * P):
        finish, bubble = simulate_programs(P, v, M, t_fwd=1.0, t_bwd=2.0)
        # bubble of interleaved 1F1B: (P - 1) / v micro-batch times out of M + (P - 1) / v
        ideal = ((P - 1) / v) / (M + (P - 1) / v)
        assert abs(bubble - ideal) < 1e-9, (P, v, M, bubble, ideal)
        assert abs(finish - 3.0 * (M * v + P - 1)) < 1e-9


def test_program_runs_every_chunk_of_every_microbatch_once_and_bounds_live_activations():
    P, v, M = 4, 2, 8
    for p in range(P):
        prog = interleaved_program(P, v, M, p)
        fwd = [e[1:] for e in prog if e[0] == "F"]
        bwd = [e[1:] for e in prog if e[0] == "B"]
        assert sorted(fwd) == sorted(bwd) == sorted((c, mb) for c in range(v) for mb in range(M))
        live = peak = 0
        for e in prog:
            live += {"F": 1, "B": -1}.get(e[0], 0)
            peak = max(peak, live)
        assert peak == min(2 * (P - p - 1) + (v - 1) * P, M * v) + 1


def test_interleave_plan_recuts_the_stages():
    plan = tiny_gpt_plan(**KW, num_gpus=(1, 2, 1), tp=[1, 2, 1], recompute=1)
    new = interleave_plan(plan, 2)
    assert new["interleave_factor"] == 2 and new["num_gpus"] == [1, 2, 1, 1, 2, 1]
    assert sum(new["num_ops_in_each_stage"]) == sum(plan["num_ops_in_each_stage"])
    assert [t[0] for t in new["model_parallel_size_of_each_op"]] == [1, 2, 1, 1, 2, 1]
    flat = lambda p: [x for s in p["recompute_ops"] for x in s]
    assert flat(new) == flat(plan)
    n = sum(plan["num_ops_in_each_stage"])
    explicit = interleave_plan(plan, 2, [5, 9, 7, 11, 13, n - 45])
    assert explicit["num_ops_in_each_stage"] == [5, 9, 7, 11, 13, n - 45] and flat(explicit) == flat(plan)
    with pytest.raises(AssertionError):
        interleave_plan(plan, 2, [5, 9, 7])
    mixed = tiny_gpt_plan(**KW, num_gpus=(2, 2), tp=[2, 1])
    mixed["model_parallel_size_of_each_op"][0][3] = 1
    with pytest.raises(AssertionError):
        interleave_plan(mixed, 2)


def _losses(plan, rank=0, world=1, steps=2, save=None):
    t = Trainer(plan, rank=rank, world_size=world, model_overrides=NODROP, lr_warmup_steps=0, device="cpu", lr=1e-3)
    out = [t.loss_value(t.train_step(gpt_batch(12, 32, 256, seed=1))) for _ in range(steps)]
    if save is not None:
        checkpointing.save_checkpoint(t, save)
        t2 = Trainer(plan, rank=rank, world_size=world, model_overrides=NODROP, lr_warmup_steps=0, device="cpu",
                     lr=1e-3, seed=99)
        assert checkpointing.load_checkpoint(t2, save) == steps
        a = t.loss_value(t.train_step(gpt_batch(12, 32, 256, seed=2)))
        b = t2.loss_value(t2.train_step(gpt_batch(12, 32, 256, seed=2)))
        assert abs(a - b) < 1e-5, (a, b)
    return out


def _worker(rank, world, plan, want, save):
    got = _losses(plan, rank, world, save=save)
    assert max(abs(a - b) for a, b in zip(got, want)) < 3e-3, (rank, got, want)


@pytest.mark.parametrize("gpus,tp,v,ckpt", [((1, 1, 1), [1, 1, 1], 2, True), ((1, 1), [1, 1], 3, False),
                                            ((1, 2, 1), [1, 2, 1], 2, False)])
def test_interleaved_training_matches_single_process(tmp_path, gpus, tp, v, ckpt):
    base = _losses(tiny_gpt_plan(**KW))
    plan = interleave_plan(tiny_gpt_plan(**KW, num_gpus=gpus, tp=tp), v)
    run_ranks(_worker, sum(gpus), plan, base, str(tmp_path / "ckpt") if ckpt else None)


def _eval_then_train(plan, rank=0, world=1):
    t = Trainer(plan, rank=rank, world_size=world, model_overrides=NODROP, lr_warmup_steps=0, device="cpu", lr=1e-3)
    batch = gpt_batch(12, 32, 256, seed=1)
    before = t.evaluate([batch, gpt_batch(12, 32, 256, seed=2)])["lm loss"]   # evaluation first: own boundaries
    losses = [t.loss_value(t.train_step(batch)) for _ in range(2)]
    after = t.evaluate([batch])["lm loss"]
    return [before] + losses + [after]


def _eval_worker(rank, world, plan, want):
    got = _eval_then_train(plan, rank, world)
    assert max(abs(a - b) for a, b in zip(got, want)) < 3e-3, (rank, got, want)


@pytest.mark.parametrize("v", [1, 2])
def test_pipeline_evaluation_matches_single_process(v):
    base = _eval_then_train(tiny_gpt_plan(**KW))
    assert base[3] < base[1]           # evaluating after two steps sees the trained weights
    plan = interleave_plan(tiny_gpt_plan(**KW, num_gpus=(1, 1), tp=[1, 1]), v)
    run_ranks(_eval_worker, 2, plan, base)


def _fuzz_worker(rank, world, plans, want):
    for i, plan in enumerate(plans):
        got = _losses(plan, rank, world)
        assert max(abs(a - b) for a, b in zip(got, want)) < 3e-3, (rank, i, got, want, plan["num_ops_in_each_stage"])


def test_interleaved_plans_with_random_cuts_match_single_process():
    """Interleaving fuzz on four ranks: two or four physical stages, 2 or 3 chunks each, virtual-stage cuts at random
    ops, one or two (tensor-parallel) GPUs per stage, recompute on or off."""
    import random
    rng = random.Random(17)
    plans = []
    for gpus, tp in (((2, 2), [2, 2]), ((1, 1, 1, 1), [1, 1, 1, 1]), ((2, 2), [1, 1])):
        v = rng.choice([2, 3]) if len(gpus) == 2 else 2
        base = tiny_gpt_plan(**KW, num_gpus=gpus, tp=tp, recompute=rng.randint(0, 1))
        n = sum(base["num_ops_in_each_stage"])
        total = len(gpus) * v
        cuts = sorted(rng.sample(range(1, n), total - 1))
        counts = [b - a for a, b in zip([0] + cuts, cuts + [n])]
        plans.append(interleave_plan(base, v, counts))
    # 12 / 2 = 6 micro-batches: a multiple of 2 stages; the 4-stage plan needs a multiple of 4 -> micro batch 3
    for p in plans:
        if len(p["num_gpus"]) // p["interleave_factor"] == 4:
            p["micro_batch_size"] = 3
    single = tiny_gpt_plan(**KW)
    want = _losses(single)
    run_ranks(_fuzz_worker, 4, [p for p in plans if p["micro_batch_size"] == 2], want, timeout=600)
    single3 = tiny_gpt_plan(**{**KW, "micro_bs": 3})
    run_ranks(_fuzz_worker, 4, [p for p in plans if p["micro_batch_size"] == 3], _losses(single3), timeout=600)


def _t5_losses(plan, rank=0, world=1):
    from superscaler_b200.data import synthetic as syn
    t = Trainer(plan, rank=rank, world_size=world, model_overrides=NODROP, lr_warmup_steps=0, device="cpu", lr=1e-3)
    b = syn.t5_batch(8, 64, 32, 256, seed=1)
    return [t.loss_value(t.train_step(b)) for _ in range(2)]


def _t5_worker(rank, world, plan, want):
    got = _t5_losses(plan, rank, world)
    assert max(abs(a - b) for a, b in zip(got, want)) < 5e-3, (rank, got, want, plan["num_ops_in_each_stage"])


def test_interleaved_t5_matches_single_process():
    """T5 with two chunks per stage and uneven cuts on 2 x 2 tensor-parallel ranks: the encoder output rides through
    the virtual stages, also across the wrap-around from the last physical stage back to the first."""
    from helpers import tiny_t5_plan
    base = tiny_t5_plan(num_gpus=(2, 2), tp=[2, 2], recompute=1, global_bs=8, micro_bs=2)
    n = sum(base["num_ops_in_each_stage"])
    plan = interleave_plan(base, 2, [9, 14, 6, n - 29])
    run_ranks(_t5_worker, 4, plan, _t5_losses(tiny_t5_plan(global_bs=8, micro_bs=2)))


def test_interleaved_wide_resnet_matches_single_process():
    """Wide-ResNet with three chunks per stage and uneven cuts (inside bottleneck blocks, so the residual rides over
    the boundaries) on two pipeline ranks, every block recomputed."""
    import test_parallel_cpu as PP
    from helpers import tiny_resnet_plan
    plan_fn = lambda **kw: tiny_resnet_plan(global_bs=16, micro_bs=4, **kw)
    base = plan_fn(num_gpus=(1, 1), recompute=1)
    n = sum(base["num_ops_in_each_stage"])
    plan = interleave_plan(base, 3, [3, 6, 9, 5, 8, n - 31])
    run_ranks(PP._resnet_fuzz_worker, 2, [plan], PP._other_model_losses("resnet", plan_fn(), steps=2), timeout=600)
