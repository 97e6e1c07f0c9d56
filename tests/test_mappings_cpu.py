"""Tensor-parallel building blocks against a single-process dense reference, for tp = 2 and 4 on CPU (gloo): the
differentiable collectives, column / row parallel linear layers, the vocabulary-parallel LM head + cross entropy,
and the dropout seed rules.  Mirrors the reference's mpu unit tests (runtime/megatron/mpu/tests/test_layers.py,
test_cross_entropy.py, test_random.py), which need one GPU per rank."""
import pytest
import torch
import torch.distributed as dist

from dist_utils import run_ranks


def _mappings_worker(rank, world):
    from superscaler_b200.parallel import mappings as M
    g = dist.group.WORLD
    torch.manual_seed(5)
    full = torch.randn(8, 4 * world, dtype=torch.float64)

    # copy_to_group: identity forward, summed gradient
    x = full.clone().requires_grad_(True)
    (M.copy_to_group(x, g) * (rank + 1)).sum().backward()
    assert torch.allclose(x.grad, torch.full_like(full, sum(range(1, world + 1))))
    # reduce_from_group: summed forward, identity backward
    x = (full * (rank + 1)).requires_grad_(True)
    y = M.reduce_from_group(x, g)
    assert torch.allclose(y, full * sum(range(1, world + 1)))
    (y * 3).sum().backward()
    assert torch.allclose(x.grad, torch.full_like(full, 3.0))
    # split <-> gather along both dims
    for dim in (0, 1):
        x = full.clone().requires_grad_(True)
        part = M.split_to_group(x, dim, g)
        assert torch.equal(part, full.chunk(world, dim)[rank])
        back = M.gather_from_group(part, dim, g)
        assert torch.equal(back, full)
        (back * torch.arange(full.numel(), dtype=torch.float64).view_as(full)).sum().backward()
        # gather's backward keeps this rank's slice of the gradient, split's backward gathers the slices again
        assert torch.allclose(x.grad, torch.arange(full.numel(), dtype=torch.float64).view_as(full))
    # reduce-scatter forward, all-gather backward
    x = (full * (rank + 1)).requires_grad_(True)
    y = M.reduce_scatter_to_group(x, 0, g)
    assert torch.allclose(y, (full * sum(range(1, world + 1))).chunk(world, 0)[rank])
    (y * (rank + 1)).sum().backward()
    want = torch.cat([torch.full((8 // world, 4 * world), float(r + 1), dtype=torch.float64) for r in range(world)])
    assert torch.allclose(x.grad, want)
    # all-to-all: rows split -> columns split, and its backward is the inverse exchange
    rows = full.chunk(world, 0)[rank].clone().requires_grad_(True)
    cols = M.all_to_all_in_group(rows, 1, 0, g)
    assert torch.equal(cols, full.chunk(world, 1)[rank])
    w = torch.arange(cols.numel(), dtype=torch.float64).view_as(cols) + 100 * rank
    (cols * w).sum().backward()
    full_w = torch.cat([torch.arange(cols.numel(), dtype=torch.float64).view_as(cols) + 100 * r for r in range(world)], 1)
    assert torch.allclose(rows.grad, full_w.chunk(world, 0)[rank])


def _linear_worker(rank, world):
    """column-parallel -> GeLU -> row-parallel (the MLP of a transformer layer) against the dense computation."""
    from superscaler_b200.parallel import mappings as M
    g = dist.group.WORLD
    torch.manual_seed(11)
    T, H, F = 12, 8, 16
    x0 = torch.randn(T, H, dtype=torch.float64)
    W1, b1 = torch.randn(F, H, dtype=torch.float64), torch.randn(F, dtype=torch.float64)
    W2, b2 = torch.randn(H, F, dtype=torch.float64), torch.randn(H, dtype=torch.float64)
    dy = torch.randn(T, H, dtype=torch.float64)

    x = x0.clone().requires_grad_(True)
    dense = [t.clone().requires_grad_(True) for t in (W1, b1, W2, b2)]
    y = torch.nn.functional.gelu(x @ dense[0].t() + dense[1], approximate="tanh") @ dense[2].t() + dense[3]
    y.backward(dy)

    xp = x0.clone().requires_grad_(True)
    w1 = W1.chunk(world, 0)[rank].clone().requires_grad_(True)      # column parallel: output features split
    bb1 = b1.chunk(world, 0)[rank].clone().requires_grad_(True)
    w2 = W2.chunk(world, 1)[rank].clone().requires_grad_(True)      # row parallel: input features split
    bb2 = b2.clone().requires_grad_(True)
    h = torch.nn.functional.gelu(M.copy_to_group(xp, g) @ w1.t() + bb1, approximate="tanh")
    yp = M.reduce_from_group(h @ w2.t(), g) + bb2
    yp.backward(dy)
    assert torch.allclose(yp, y, atol=1e-10)
    assert torch.allclose(xp.grad, x.grad, atol=1e-10)
    assert torch.allclose(w1.grad, dense[0].grad.chunk(world, 0)[rank], atol=1e-10)
    assert torch.allclose(bb1.grad, dense[1].grad.chunk(world, 0)[rank], atol=1e-10)
    assert torch.allclose(w2.grad, dense[2].grad.chunk(world, 1)[rank], atol=1e-10)
    assert torch.allclose(bb2.grad, dense[3].grad, atol=1e-10)


def _ce_worker(rank, world):
    """Vocabulary-parallel LM head + cross entropy (max / sum-exp / target-logit reductions over the group) against
    F.cross_entropy on the full logits, with a loss mask."""
    from superscaler_b200.ops import functional as F
    g = dist.group.WORLD
    torch.manual_seed(3)
    T, H, V = 24, 16, 32 * world
    x0 = torch.randn(T, H)
    W = torch.randn(V, H) * 0.5
    tgt = torch.randint(0, V, (T,))
    mask = (torch.rand(T) > 0.3).float()

    x = x0.clone().requires_grad_(True)
    Wd = W.clone().requires_grad_(True)
    ref = (torch.nn.functional.cross_entropy(x @ Wd.t(), tgt, reduction="none") * mask).sum() * 0.125
    ref.backward()

    v_local = V // world
    xp = x0.clone().requires_grad_(True)
    wl = W[rank * v_local:(rank + 1) * v_local].clone().requires_grad_(True)
    loss = F.lm_head_cross_entropy(xp, wl, tgt, mask, rank * v_local, 0.125, g)
    loss.backward()
    # the head emulates the kernels' bf16 logits and bf16 GEMM outputs on the CPU: tolerances are bf16-sized
    assert abs(float(loss.detach()) - float(ref.detach())) < 2e-3 * abs(float(ref.detach()))
    gx = xp.grad.float().clone()
    dist.all_reduce(gx)          # every rank holds its vocabulary shard's share of dx
    rel = lambda a, b: float((a.float() - b).norm() / b.norm())
    assert rel(gx, x.grad) < 2e-2
    assert rel(wl.grad, Wd.grad[rank * v_local:(rank + 1) * v_local]) < 2e-2


def _seed_worker(rank, world):
    """Dropout seeds: equal inside a tensor-parallel group for replicated tensors, different for sharded ones,
    different across data-parallel ranks; the counter state can be saved and replayed."""
    from superscaler_b200.models.base import Env, Op, OpInfo
    from superscaler_b200.ops import functional as F
    from superscaler_b200.parallel.state import ParallelState
    ps = ParallelState([world], rank, world)
    ps.ensure_groups(ps.all_op_groups([[(2, world // 2)]]))
    env = Env(cfg=None, pstate=ps, store=None, micro_bs=world)
    op = Op(OpInfo(name="x", index=0, layer=0, tp=2, dp=world // 2, algo=0, recompute=0), env)
    F.manual_seed(99)
    state = F.seed_state().get_state()
    rep, shard = op.seed(), op.seed(sharded=True)
    F.seed_state().set_state(state)
    assert (op.seed(), op.seed(sharded=True)) == (rep, shard)      # replay
    got = [None] * world
    dist.all_gather_object(got, (op.pl.tp_rank, op.pl.dp_rank, rep, shard))
    for tp_a, dp_a, rep_a, sh_a in got:
        for tp_b, dp_b, rep_b, sh_b in got:
            if (tp_a, dp_a) == (tp_b, dp_b):
                continue
            if dp_a == dp_b:
                assert rep_a == rep_b and sh_a != sh_b
            else:
                assert rep_a != rep_b and sh_a != sh_b


@pytest.mark.parametrize("world", [2, 4])
def test_differentiable_collectives(world):
    run_ranks(_mappings_worker, world)


@pytest.mark.parametrize("world", [2, 4])
def test_column_and_row_parallel_linear_match_dense(world):
    run_ranks(_linear_worker, world)


@pytest.mark.parametrize("world", [2, 4])
def test_vocab_parallel_cross_entropy_matches_dense(world):
    run_ranks(_ce_worker, world)


def test_dropout_seed_rules():
    run_ranks(_seed_worker, 4)
