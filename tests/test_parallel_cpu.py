"""Multi-rank training on CPU (gloo): pipeline, tensor and data parallel plans must reproduce the losses of
the single-process run of the same model (constant seed, dropout off) -- the DEBUG_FIX_WEIGHT-style
cross-configuration check of the reference (runtime/megatron/training.py:215-217)."""
import pytest
import torch

from superscaler_b200.data.synthetic import gpt_batch
from superscaler_b200.runtime.trainer import Trainer

from dist_utils import run_ranks
from helpers import tiny_gpt_plan

NODROP = dict(hidden_dropout=0.0, attention_dropout=0.0, max_tp=2)
KW = dict(layers=2, seq=64, hidden=64, heads=2, head_dim=32, vocab=256, global_bs=8, micro_bs=4)


def _losses(plan, rank=0, world=1, steps=3):
    t = Trainer(plan, rank=rank, world_size=world, model_overrides=NODROP, lr_warmup_steps=0, device="cpu", lr=1e-3)
    out = []
    for _ in range(steps):
        out.append(t.loss_value(t.train_step(gpt_batch(8, 64, 256, seed=1))))
    return out


def _worker(rank, world, plan, want):
    got = _losses(plan, rank, world)
    assert max(abs(a - b) for a, b in zip(got, want)) < 3e-3, (rank, got, want)


BASE = None


def _base():
    global BASE
    if BASE is None:
        BASE = _losses(tiny_gpt_plan(**KW))
    return BASE


@pytest.mark.parametrize("name,plan_kw,world", [
    ("dp2", dict(num_gpus=(2,), tp=[1]), 2),
    ("tp2", dict(num_gpus=(2,), tp=[2]), 2),
    ("pp2", dict(num_gpus=(1, 1)), 2),
    ("pp2_tp2_dp2", dict(num_gpus=(2, 2), tp=[2, 1]), 4),
    ("pp3_uneven", dict(num_gpus=(1, 2, 1), tp=[1, 2, 1], ops_per_stage=[9, 12, 8]), 4),
])
def test_parallel_plans_match_single_process(name, plan_kw, world):
    plan = tiny_gpt_plan(**KW, **plan_kw)
    run_ranks(_worker, world, plan, _base())


def test_in_stage_resharding_matches_single_process():
    # one stage of 2 GPUs whose ops switch from tp2 to dp2 in the middle of a layer and back
    plan = tiny_gpt_plan(**KW, num_gpus=(2,), tp=[2])
    n = plan["num_ops_in_each_stage"][0]
    tp = [2] * n
    for i in range(9, 20):
        tp[i] = 1
    plan["model_parallel_size_of_each_op"] = [tp]
    plan["data_parallel_size_of_each_op"] = [[2 // t for t in tp]]
    plan["resharding_stages"] = [True]
    run_ranks(_worker, 2, plan, _base())


def _other_model_losses(model, plan, rank=0, world=1, steps=3):
    from superscaler_b200.data import synthetic as syn
    if model == "t5":
        ov, batch = dict(hidden_dropout=0.0, attention_dropout=0.0, max_tp=2), syn.t5_batch(4, 64, 32, 256, seed=1)
    else:
        ov, batch = dict(image_size=64, num_classes=16), syn.resnet_batch(16, 64, 16, seed=1, dtype=torch.float32)
    t = Trainer(plan, rank=rank, world_size=world, model_overrides=ov, lr_warmup_steps=0, device="cpu", lr=1e-3)
    return [t.loss_value(t.train_step(batch)) for _ in range(steps)]


def _other_model_worker(rank, world, model, plan, want):
    got = _other_model_losses(model, plan, rank, world)
    # the ResNet bound covers what threaded fp32 reductions plus Adam do to two runs of the SAME plan (3e-3)
    bound = 5e-3 if model == "t5" else 2e-2 * max(1.0, abs(want[0]))
    assert max(abs(a - b) for a, b in zip(got, want)) < bound, (rank, got, want)


# Data-parallel Wide-ResNet plans are left out on purpose: BatchNorm normalises with the statistics of the samples a
# rank sees (as torch's BatchNorm2d does in the reference), so splitting the micro-batch changes the function.
@pytest.mark.parametrize("model,plan_kw,world", [
    ("t5", dict(num_gpus=(2,), tp=[2]), 2), ("t5", dict(num_gpus=(2,), tp=[1]), 2), ("t5", dict(num_gpus=(1, 1)), 2),
    ("t5", dict(num_gpus=(1, 2, 1), tp=[1, 2, 1]), 4),
    ("resnet", dict(num_gpus=(2,), tp=[2]), 2), ("resnet", dict(num_gpus=(1, 1)), 2),
    ("resnet", dict(num_gpus=(2, 2), tp=[2, 2]), 4),
])
def test_t5_and_resnet_parallel_plans_match_single_process(model, plan_kw, world):
    from helpers import tiny_resnet_plan, tiny_t5_plan
    plan_fn = tiny_t5_plan if model == "t5" else (lambda **kw: tiny_resnet_plan(global_bs=16, micro_bs=8, **kw))
    base = _other_model_losses(model, plan_fn())
    run_ranks(_other_model_worker, world, model, plan_fn(**plan_kw), base)


def test_gpt_alternative_partitioning_matches_single_process():
    """algo 1 of every tensor-parallel op (row-parallel QKV and MLP up-projection, column-parallel output
    projections) on two ranks, alone and mixed with algo 0 from layer to layer."""
    plan = tiny_gpt_plan(**KW, num_gpus=(2,), tp=[2])
    n = plan["num_ops_in_each_stage"][0]
    plan["algo_of_each_op"] = [[1] * n]
    plan["resharding_stages"] = [True]
    run_ranks(_worker, 2, plan, _base())
    mixed = tiny_gpt_plan(**KW, num_gpus=(2,), tp=[2])
    mixed["algo_of_each_op"] = [[(i // 13) % 2 for i in range(n)]]
    mixed["resharding_stages"] = [True]
    run_ranks(_worker, 2, mixed, _base())


def test_resnet_input_channel_partitioning_matches_single_process():
    """algo 1 of the convolutions (input channels split, partial outputs summed) on two ranks."""
    from helpers import tiny_resnet_plan
    plan_fn = lambda **kw: tiny_resnet_plan(global_bs=16, micro_bs=8, **kw)
    base = _other_model_losses("resnet", plan_fn())
    plan = plan_fn(num_gpus=(2,), tp=[2])
    n = plan["num_ops_in_each_stage"][0]
    plan["algo_of_each_op"] = [[1] * n]
    plan["resharding_stages"] = [True]
    run_ranks(_other_model_worker, 2, "resnet", plan, base)


@pytest.mark.parametrize("plan_kw,world", [(dict(num_gpus=(2,), tp=[2]), 2), (dict(num_gpus=(1, 1)), 2),
                                           (dict(num_gpus=(2,), tp=[1]), 2)])
def test_recompute_under_parallel_plans_matches_single_process(plan_kw, world):
    """Per-op recompute (every layer checkpointed) combined with tensor, pipeline and data parallelism."""
    run_ranks(_worker, world, tiny_gpt_plan(**KW, recompute=1, **plan_kw), _base())


def _searched_resnet_worker(rank, world, plan):
    from superscaler_b200.data import synthetic as syn
    t = Trainer(plan, rank=rank, world_size=world, lr_warmup_steps=0, device="cpu", lr=1e-3,
                model_overrides=dict(image_size=64, num_classes=16, in_channels=8))
    batch = syn.resnet_batch(16, 64, 16, seed=1, dtype=torch.float32)
    losses = [t.loss_value(t.train_step(batch)) for _ in range(3)]
    assert all(l == l for l in losses) and losses[-1] < losses[0], losses


def test_runtime_executes_the_plan_the_search_wrote_for_wide_resnet():
    """The 2-stage plan of the reference search for Wide-ResNet 1B on 4 GPUs (stage 1 switches from dp 2 to tp 2
    in the middle, both partitioning algorithms, partial recompute), run with narrow channels on four gloo ranks."""
    import json
    import os
    with open(os.path.join(os.path.dirname(__file__), "golden", "reference_search", "resnet_1B_2stages.json")) as f:
        plan = json.load(f)
    plan.update(global_batch_size=16, micro_batch_size=8, in_channels=8)
    run_ranks(_searched_resnet_worker, 4, plan)


def _searched_gpt_losses(plan, rank=0, world=1):
    t = Trainer(plan, rank=rank, world_size=world, model_overrides=NODROP, lr_warmup_steps=0, device="cpu", lr=1e-3)
    return [t.loss_value(t.train_step(gpt_batch(8, 32, 256, seed=1))) for _ in range(2)]


def _searched_gpt_worker(rank, world, plan, want):
    got = _searched_gpt_losses(plan, rank, world)
    assert max(abs(a - b) for a, b in zip(got, want)) < 5e-3, (rank, got, want)


@pytest.mark.parametrize("stages", [2, 4])
def test_runtime_executes_the_plans_the_search_wrote_for_gpt(stages):
    """The reference search's GPT-3 1.3B plans for 4 GPUs (uneven op counts per stage, partial recompute chosen
    per op; the 2-stage plan with two GPUs per stage), shrunk to a narrow 24-layer model, against one process."""
    import json
    import os
    with open(os.path.join(os.path.dirname(__file__), "golden", "reference_search", f"gpt_1_3B_{stages}stages.json")) as f:
        plan = json.load(f)
    plan.update(global_batch_size=8, micro_batch_size=2, seq_length=32, max_position_embeddings=32, hidden_size=64,
                num_attention_heads=2, kv_channels=32, vocab_size=256)
    if max(max(d) for d in plan["data_parallel_size_of_each_op"]) > 2:
        plan["micro_batch_size"] = 4
    single = tiny_gpt_plan(layers=24, seq=32, hidden=64, heads=2, head_dim=32, vocab=256, global_bs=8,
                           micro_bs=plan["micro_batch_size"])
    run_ranks(_searched_gpt_worker, 4, plan, _searched_gpt_losses(single))


def _searched_t5_losses(plan, rank=0, world=1):
    from superscaler_b200.data import synthetic as syn
    t = Trainer(plan, rank=rank, world_size=world, model_overrides=NODROP, lr_warmup_steps=0, device="cpu", lr=1e-3)
    return [t.loss_value(t.train_step(syn.t5_batch(8, 32, 16, 256, seed=1))) for _ in range(2)]


def _searched_t5_worker(rank, world, plan, want):
    got = _searched_t5_losses(plan, rank, world)
    assert max(abs(a - b) for a, b in zip(got, want)) < 5e-3, (rank, got, want)


def test_runtime_executes_the_plan_the_search_wrote_for_t5():
    """The reference search's 4-stage T5 770M plan (ops per stage 113 / 118 / 195 / 395: the encoder output crosses
    three boundaries as an extra tensor), shrunk to a narrow 24 + 24 layer model."""
    import json
    import os
    from helpers import tiny_t5_plan
    with open(os.path.join(os.path.dirname(__file__), "golden", "reference_search", "t5_770M_4stages.json")) as f:
        plan = json.load(f)
    small = dict(global_batch_size=8, micro_batch_size=2, encoder_seq_length=32, decoder_seq_length=16,
                 max_position_embeddings=32, hidden_size=64, num_attention_heads=2, kv_channels=32, ffn_hidden_size=128,
                 vocab_size=256)
    plan.update(small)
    single = tiny_t5_plan(layers=24, enc_seq=32, dec_seq=16, hidden=64, heads=2, head_dim=32, ffn=128, vocab=256,
                          global_bs=8, micro_bs=2)
    run_ranks(_searched_t5_worker, 4, plan, _searched_t5_losses(single), timeout=600)


def test_runtime_executes_the_estimated_13b_plan_shape():
    """plans/gpt_13B_8gpu_b200_extrapolated.json (two pipeline stages of four data-parallel GPUs, searched against
    scaled tables) with narrow layers on eight gloo ranks, against one process."""
    import json
    import os
    path = os.path.join(os.path.dirname(os.path.dirname(__file__)), "plans", "gpt_13B_8gpu_b200_extrapolated.json")
    with open(path) as f:
        plan = json.load(f)
    assert sum(plan["num_gpus"]) == 8 and plan["num_layers"] == 40
    plan.update(global_batch_size=8, micro_batch_size=4, seq_length=32, max_position_embeddings=32, hidden_size=64,
                num_attention_heads=2, kv_channels=32, vocab_size=256)
    single = tiny_gpt_plan(layers=40, seq=32, hidden=64, heads=2, head_dim=32, vocab=256, global_bs=8, micro_bs=4)
    run_ranks(_searched_gpt_worker, 8, plan, _searched_gpt_losses(single), timeout=600)


def _fuzz_worker(rank, world, plans, want):
    for i, plan in enumerate(plans):
        got = _losses(plan, rank, world)
        assert max(abs(a - b) for a, b in zip(got, want)) < 3e-3, (rank, i, got, want,
                                                                    plan["model_parallel_size_of_each_op"],
                                                                    plan["algo_of_each_op"])


@pytest.mark.parametrize("seed", [0, 1])
def test_random_per_op_layouts_match_single_process(seed):
    """In-stage resharding fuzz: every op of a two-rank stage draws its own (tp, dp) in {(1, 2), (2, 1)} in runs of
    random length and its own partitioning algorithm; forward AND gradients (the later losses) must not change."""
    import random
    rng = random.Random(seed)
    plans = []
    for _ in range(4):
        plan = tiny_gpt_plan(**KW, num_gpus=(2,), tp=[2])
        n = plan["num_ops_in_each_stage"][0]
        tp, cur = [], rng.choice([1, 2])
        while len(tp) < n:
            tp += [cur] * rng.randint(1, 9)
            cur = 3 - cur
        tp = tp[:n]
        plan["model_parallel_size_of_each_op"] = [tp]
        plan["data_parallel_size_of_each_op"] = [[2 // t for t in tp]]
        plan["algo_of_each_op"] = [[rng.randint(0, 1) for _ in range(n)]]
        plan["resharding_stages"] = [True]
        rc, cur = [], rng.randint(0, 1)          # and its own recompute flag, in runs of random length
        while len(rc) < n:
            rc += [cur] * rng.randint(1, 7)
            cur = 1 - cur
        plan["recompute_ops"] = [rc[:n]]
        plans.append(plan)
    run_ranks(_fuzz_worker, 2, plans, _base(), timeout=600)


def _fuzz4_losses(plan, rank=0, world=1):
    ov = dict(hidden_dropout=0.0, attention_dropout=0.0, max_tp=4)
    t = Trainer(plan, rank=rank, world_size=world, model_overrides=ov, lr_warmup_steps=0, device="cpu", lr=1e-3)
    return [t.loss_value(t.train_step(gpt_batch(8, 64, 256, seed=1))) for _ in range(2)]


def _fuzz4_worker(rank, world, plans, want):
    for i, plan in enumerate(plans):
        got = _fuzz4_losses(plan, rank, world)
        assert max(abs(a - b) for a, b in zip(got, want)) < 3e-3, (rank, i, got, want,
                                                                    plan["model_parallel_size_of_each_op"],
                                                                    plan["algo_of_each_op"])


def test_random_per_op_layouts_on_four_ranks_match_single_process():
    """The same fuzz with tp in {1, 2, 4} on a four-rank stage (dp = 4 / tp), four heads."""
    import random
    rng = random.Random(7)
    kw = dict(layers=2, seq=64, hidden=64, heads=4, head_dim=16, vocab=256, global_bs=8, micro_bs=4)
    plans = []
    for _ in range(3):
        plan = tiny_gpt_plan(**kw, num_gpus=(4,), tp=[4])
        n = plan["num_ops_in_each_stage"][0]
        tp = []
        while len(tp) < n:
            tp += [rng.choice([1, 2, 4])] * rng.randint(1, 9)
        tp = tp[:n]
        plan["model_parallel_size_of_each_op"] = [tp]
        plan["data_parallel_size_of_each_op"] = [[4 // t for t in tp]]
        plan["algo_of_each_op"] = [[rng.randint(0, 1) for _ in range(n)]]
        plan["resharding_stages"] = [True]
        plans.append(plan)
    run_ranks(_fuzz4_worker, 4, plans, _fuzz4_losses(tiny_gpt_plan(**kw)), timeout=600)


def _resnet_fuzz_worker(rank, world, plans, want):
    for i, plan in enumerate(plans):
        got = _other_model_losses("resnet", plan, rank, world, steps=2)
        assert max(abs(a - b) for a, b in zip(got, want)) < 2e-2 * max(1.0, abs(want[0])), \
            (rank, i, got, want, plan["model_parallel_size_of_each_op"], plan["algo_of_each_op"])


def test_random_per_op_layouts_of_wide_resnet_match_single_process():
    """Convolutions, ReLU and pooling ops draw (tp, dp) and the partitioning algorithm at random on two ranks;
    the ops that normalise over the batch (BatchNorm, and the downsample path that contains one) stay on dp = 1 so
    that their statistics see the whole micro-batch, as in the single-process run."""
    import random
    from helpers import tiny_resnet_plan
    from superscaler_b200.models.resnet import ResNetConfig, resnet_op_names
    rng = random.Random(3)
    plan_fn = lambda **kw: tiny_resnet_plan(global_bs=16, micro_bs=8, **kw)
    names = resnet_op_names(ResNetConfig(blocks=(1, 1, 1, 1)))
    plans = []
    for _ in range(3):
        plan = plan_fn(num_gpus=(2,), tp=[2])
        assert plan["num_ops_in_each_stage"][0] == len(names)
        tp = [2 if ("bn" in n or "downsample" in n) else rng.choice([1, 2]) for n in names]
        plan["model_parallel_size_of_each_op"] = [tp]
        plan["data_parallel_size_of_each_op"] = [[2 // t for t in tp]]
        plan["algo_of_each_op"] = [[rng.randint(0, 1) for _ in names]]
        plan["resharding_stages"] = [True]
        plans.append(plan)
    base = _other_model_losses("resnet", plan_fn(), steps=2)
    run_ranks(_resnet_fuzz_worker, 2, plans, base, timeout=600)


def test_random_stage_cuts_match_single_process():
    """Pipeline fuzz on four ranks: 2 to 4 stages cut at random ops (also in the middle of a layer, where the
    residual, the deferred bias or the value tensor cross the boundary), random GPU counts and tp per stage,
    recompute on or off per stage."""
    import random
    rng = random.Random(5)
    kw = dict(layers=2, seq=64, hidden=64, heads=4, head_dim=16, vocab=256, global_bs=8, micro_bs=4)
    n = len(tiny_gpt_plan(**kw)["algo_of_each_op"][0])
    plans = []
    for _ in range(4):
        stages = rng.randint(2, 4)
        gpus = {2: [(2, 2), (1, 3), (3, 1)], 3: [(1, 1, 2), (2, 1, 1), (1, 2, 1)], 4: [(1, 1, 1, 1)]}[stages]
        gpus = [g for g in gpus if all(x in (1, 2, 4) for x in g)] or [(2, 2)]
        num_gpus = rng.choice(gpus)
        cuts = sorted(rng.sample(range(1, n), stages - 1))
        counts = [b - a for a, b in zip([0] + cuts, cuts + [n])]
        tp = [rng.choice([t for t in (1, 2, 4) if t <= g]) for g in num_gpus]
        plan = tiny_gpt_plan(**kw, num_gpus=num_gpus, tp=tp, ops_per_stage=counts, recompute=rng.randint(0, 1))
        plans.append(plan)
    run_ranks(_fuzz4_worker, 4, plans, _fuzz4_losses(tiny_gpt_plan(**kw)), timeout=600)


def _t5_fuzz_worker(rank, world, plans, want):
    for i, plan in enumerate(plans):
        got = _other_model_losses("t5", plan, rank, world, steps=2)
        assert max(abs(a - b) for a, b in zip(got, want)) < 5e-3, (rank, i, got, want, plan["num_ops_in_each_stage"])


def test_random_stage_cuts_of_t5_match_single_process():
    """T5 on four ranks with cuts at random ops: the encoder output travels as an extra tensor through every stage
    between its producer and the last cross-attention that reads it."""
    import random
    from helpers import tiny_t5_plan
    rng = random.Random(11)
    n = len(tiny_t5_plan()["algo_of_each_op"][0])
    plans = []
    for num_gpus in ((1, 1, 1, 1), (2, 1, 1), (1, 1, 2)):
        stages = len(num_gpus)
        cuts = sorted(rng.sample(range(1, n), stages - 1))
        counts = [b - a for a, b in zip([0] + cuts, cuts + [n])]
        tp = [rng.choice([t for t in (1, 2) if t <= g]) for g in num_gpus]
        plans.append(tiny_t5_plan(num_gpus=num_gpus, tp=tp, ops_per_stage=counts, recompute=rng.randint(0, 1)))
    run_ranks(_t5_fuzz_worker, 4, plans, _other_model_losses("t5", tiny_t5_plan(), steps=2), timeout=600)


def test_random_stage_cuts_of_wide_resnet_match_single_process():
    """Wide-ResNet on four ranks, cuts at random ops (inside bottleneck blocks too, where the block input travels on
    as the residual), stages of one GPU or of two tensor-parallel GPUs."""
    import random
    from helpers import tiny_resnet_plan
    rng = random.Random(13)
    plan_fn = lambda **kw: tiny_resnet_plan(global_bs=16, micro_bs=8, **kw)
    n = len(plan_fn()["algo_of_each_op"][0])
    plans = []
    for num_gpus in ((1, 1, 1, 1), (2, 1, 1), (1, 2, 1), (2, 2)):
        stages = len(num_gpus)
        cuts = sorted(rng.sample(range(1, n), stages - 1))
        counts = [b - a for a, b in zip([0] + cuts, cuts + [n])]
        plan = plan_fn(num_gpus=num_gpus, tp=list(num_gpus), ops_per_stage=counts, recompute=rng.randint(0, 1))
        plan["algo_of_each_op"] = [[rng.randint(0, 1) for _ in range(c)] for c in counts]
        plan["resharding_stages"] = [True] * stages
        plans.append(plan)
    base = _other_model_losses("resnet", plan_fn(), steps=2)
    run_ranks(_resnet_fuzz_worker, 4, plans, base, timeout=600)


def test_ranks_on_different_nodes_are_told_apart(monkeypatch):
    """Peer-mapped buffers are only used inside a node: with LOCAL_WORLD_SIZE ranks per node, rank sets that cross a
    node boundary are reported as such (tensor-parallel groups and the data-parallel gradient buffer then use NCCL)."""
    from superscaler_b200.parallel.state import ParallelState
    ps = ParallelState([4], rank=0, world_size=4)
    monkeypatch.setenv("LOCAL_WORLD_SIZE", "2")
    assert ps.same_node([0, 1]) and ps.same_node([2, 3]) and not ps.same_node([1, 2]) and not ps.same_node(range(4))
    monkeypatch.setenv("LOCAL_WORLD_SIZE", "4")
    assert ps.same_node(range(4))
    monkeypatch.delenv("LOCAL_WORLD_SIZE")
    assert ps.same_node(range(4))


def _saved_bytes_worker(rank, world, plan, want):
    """Losses as in the single-process run, with and without the 1 / tp shares; bytes kept by the recompute
    segments for the backward pass are counted through autograd's saved-tensor hooks."""
    kept = {}
    for share in (False, True):
        t = Trainer(plan, rank=rank, world_size=world, model_overrides=NODROP, lr_warmup_steps=0, device="cpu", lr=1e-3,
                    distribute_checkpointed_activations=share)
        total = [0]

        def pack(x, total=total):
            total[0] += x.numel() * x.element_size()
            return x

        batch = t.to_device(gpt_batch(8, 64, 256, seed=1))
        with torch.autograd.graph.saved_tensors_hooks(pack, lambda x: x):
            t.forward_backward(batch)
        kept[share] = total[0]
        t._fold_autograd_grads()
        t.store.zero_grad()
        got = [t.loss_value(t.train_step(gpt_batch(8, 64, 256, seed=1))) for _ in range(3)]
        assert max(abs(a - b) for a, b in zip(got, want)) < 3e-3, (rank, share, got, want)
    # each of the two layers keeps x [4 x 64 rows, 64] in bf16 per micro-batch: half of it with the shares
    full_inputs = 2 * 2 * (4 * 64 * 64 * 2)
    assert kept[False] - kept[True] == full_inputs // 2, (kept, full_inputs)


def test_recompute_segments_keep_one_share_of_replicated_inputs_per_tensor_parallel_rank():
    run_ranks(_saved_bytes_worker, 2, tiny_gpt_plan(**KW, recompute=1, num_gpus=(2,), tp=[2]), _base())


def _shares_worker(rank, world, plan, want):
    t = Trainer(plan, rank=rank, world_size=world, model_overrides=NODROP, lr_warmup_steps=0, device="cpu", lr=1e-3,
                distribute_checkpointed_activations=True)
    got = [t.loss_value(t.train_step(gpt_batch(8, 64, 256, seed=1))) for _ in range(3)]
    assert max(abs(a - b) for a, b in zip(got, want)) < 3e-3, (rank, got, want)


def test_shares_of_saved_inputs_in_a_pipeline_with_a_tensor_parallel_stage():
    plan = tiny_gpt_plan(**KW, recompute=1, num_gpus=(1, 2, 1), tp=[1, 2, 1], ops_per_stage=[9, 12, 8])
    run_ranks(_shares_worker, 4, plan, _base())


def _norm_worker(rank, world, plan, want):
    t = Trainer(plan, rank=rank, world_size=world, model_overrides=NODROP, lr_warmup_steps=0, device="cpu",
                shard_optimizer=False)
    assert abs(t.optimizer.params_norm() - want) < 1e-4 * want, (rank, t.optimizer.params_norm(), want)
    t.store.grad.fill_(0.0)
    total = sum(n for _, n in Trainer(tiny_gpt_plan(**KW), device="cpu", model_overrides=NODROP).store.offsets.values())
    assert t.optimizer.count_zeros_in_grad() == total          # every entry of the whole model, each counted once


@pytest.mark.parametrize("plan_kw,world", [(dict(num_gpus=(2,), tp=[2]), 2), (dict(num_gpus=(2,), tp=[1]), 2),
                                           (dict(num_gpus=(1, 1)), 2)])
def test_parameter_norm_and_zero_count_cover_the_model_once(plan_kw, world):
    base = Trainer(tiny_gpt_plan(**KW), device="cpu", model_overrides=NODROP)
    run_ranks(_norm_worker, world, tiny_gpt_plan(**KW, **plan_kw), base.optimizer.params_norm())
