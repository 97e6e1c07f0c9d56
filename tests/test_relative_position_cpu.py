"""T5 relative-position buckets against the definition in the `transformers` package, and the distance-table form
a kernel consumes."""
import pytest
import torch

from superscaler_b200.models.relative_position import bias_from_table, distance_table, relative_position_bucket


@pytest.mark.parametrize("bidirectional", [True, False])
@pytest.mark.parametrize("buckets,max_distance", [(32, 128), (16, 64), (32, 20)])
def test_buckets_match_transformers(bidirectional, buckets, max_distance):
    t5 = pytest.importorskip("transformers.models.t5.modeling_t5")
    d = torch.arange(-700, 701)
    want = t5.T5Attention._relative_position_bucket(d, bidirectional=bidirectional, num_buckets=buckets,
                                                    max_distance=max_distance)
    got = relative_position_bucket(d, bidirectional, buckets, max_distance)
    assert torch.equal(got, want)
    assert int(got.min()) >= 0 and int(got.max()) < buckets


def test_distance_table_expands_to_the_full_bias_and_carries_gradients():
    torch.manual_seed(0)
    heads, buckets, sq, sk = 3, 32, 40, 56
    w = torch.randn(heads, buckets, requires_grad=True)
    for bidirectional in (True, False):
        table = distance_table(w, sq, sk, bidirectional)
        assert table.shape == (heads, sq + sk - 1)
        bias = bias_from_table(table, sq, sk)
        q, k = torch.arange(sq)[:, None], torch.arange(sk)[None, :]
        want = w[:, relative_position_bucket(k - q, bidirectional)]
        assert torch.equal(bias, want)
    g = torch.randn(heads, sq, sk)
    (bias_from_table(distance_table(w, sq, sk, True), sq, sk) * g).sum().backward()
    want = torch.zeros(heads, buckets)
    b = relative_position_bucket(k - q, True)
    for h in range(heads):
        want[h].index_add_(0, b.reshape(-1), g[h].reshape(-1))
    assert torch.allclose(w.grad, want, atol=1e-4)


def _t5_losses(plan, rank=0, world=1, fuse=True, steps=3):
    from superscaler_b200.data.synthetic import t5_batch
    from superscaler_b200.runtime.trainer import Trainer
    ov = dict(hidden_dropout=0.0, attention_dropout=0.0, relative_position_bias=True, max_tp=2)
    t = Trainer(plan, rank=rank, world_size=world, model_overrides=ov, fuse=fuse, lr_warmup_steps=0, device="cpu",
                lr=2e-3)
    names = [n for n in t.store.params if "relative_attention_bias" in n]
    before = {n: t.store.params[n].detach().clone() for n in names}
    out = [t.loss_value(t.train_step(t5_batch(4, 64, 32, 256, seed=1))) for _ in range(steps)]
    tables = {n: (before[n], t.store.params[n].detach().clone()) for n in names}
    return out, tables, t


def _t5_worker(rank, world, plan, want):
    got, _, _ = _t5_losses(plan, rank, world)
    assert max(abs(a - b) for a, b in zip(got, want)) < 6e-3, (rank, got, want)


def test_t5_with_relative_position_bias_trains_and_matches_across_plans():
    import sys, os
    sys.path.insert(0, os.path.dirname(__file__))
    from dist_utils import run_ranks
    from helpers import tiny_t5_plan
    fused, tables, t = _t5_losses(tiny_t5_plan(layers=2))
    # one table per stack, shared by both layers, and it learns
    assert len(tables) == 2 and all(a.shape == (2, 32) for a, _ in tables.values())
    assert all(not torch.equal(a, b) for a, b in tables.values())
    assert fused[-1] < fused[0]
    unfused, _, _ = _t5_losses(tiny_t5_plan(layers=2), fuse=False)
    assert max(abs(a - b) for a, b in zip(fused, unfused)) < 2e-3
    # tensor parallel (heads split) and pipeline parallel (the decoder table's holder sits in a later stage)
    run_ranks(_t5_worker, 2, tiny_t5_plan(layers=2, num_gpus=(2,), tp=[2]), fused)
    run_ranks(_t5_worker, 2, tiny_t5_plan(layers=2, num_gpus=(1, 1)), fused)
