"""Single-process runtime tests on CPU (plain PyTorch restatements of the kernels)."""
import pytest
import torch

from superscaler_b200.data.synthetic import gpt_batch
from superscaler_b200.runtime.lr import LRSchedule
from superscaler_b200.runtime.trainer import Trainer

from helpers import tiny_gpt_plan

NODROP = dict(hidden_dropout=0.0, attention_dropout=0.0, max_tp=1)


def _run(plan, steps=3, **kw):
    t = Trainer(plan, model_overrides=NODROP, lr_warmup_steps=0, device="cpu", **kw)
    out = []
    for _ in range(steps):
        out.append(t.loss_value(t.train_step(gpt_batch(plan["global_batch_size"], plan["seq_length"], 512, seed=1))))
    return out, t


def test_tiny_gpt_trains_and_variants_agree():
    base, t = _run(tiny_gpt_plan())
    assert base[-1] < base[0] and abs(base[0] - 6.24) < 0.1
    unfused, _ = _run(tiny_gpt_plan(), fuse=False)
    recomp, _ = _run(tiny_gpt_plan(recompute=1))
    recomp_unfused, _ = _run(tiny_gpt_plan(recompute=1), fuse=False)
    for other in (unfused, recomp, recomp_unfused):
        assert max(abs(a - b) for a, b in zip(base, other)) < 2e-3
    names = [type(o).__name__ for o in t.stage.ops]
    assert "FusedAttention" in names and "FusedMLP" in names and "FusedDenseDropAdd" in names


def test_microbatching_is_equivalent():
    a, _ = _run(tiny_gpt_plan(global_bs=4, micro_bs=4))
    b, _ = _run(tiny_gpt_plan(global_bs=4, micro_bs=1))
    assert max(abs(x - y) for x, y in zip(a, b)) < 2e-3


def test_recompute_segments_break_at_layers():
    _, t = _run(tiny_gpt_plan(recompute=1), steps=1)
    segs = t.stage.segments
    assert [s.recompute for s in segs] == [False, True, True, False]
    assert segs[1].ops[0].info.name == "enc-1st-layernorm" and segs[2].ops[0].info.name == "enc-1st-layernorm"


def test_lr_schedule():
    s = LRSchedule(1.0, 0.1, warmup_steps=10, decay_steps=110, style="cosine")
    lrs = [s.step() for _ in range(120)]
    assert abs(lrs[4] - 0.5) < 1e-9 and abs(lrs[9] - 1.0) < 1e-9
    assert abs(lrs[59] - 0.55) < 1e-6 and lrs[-1] == 0.1
    sd = s.state_dict()
    s2 = LRSchedule(2.0, 0.0, 1, 2)
    s2.load_state_dict(sd)
    assert s2.get_lr() == s.get_lr()
    lin = LRSchedule(1.0, 0.0, warmup_steps=0, decay_steps=100, style="linear")
    assert abs(lin.step(50) - 0.5) < 1e-9


def test_memory_buffers_and_reports():
    import torch
    from superscaler_b200.runtime.memory import MemoryBuffer, RingMemBuffer, debug_mem_report, report_memory
    buf = MemoryBuffer("act", 64, torch.float32, track_usage=True, device="cpu")
    a = buf.get((4, 4))
    b = buf.add(torch.arange(8, dtype=torch.float32))
    assert a.shape == (4, 4) and b.tolist() == list(range(8)) and buf.numel_in_use() == 24
    assert a.data_ptr() == buf.data.data_ptr() and b.data_ptr() == buf.data[16:].data_ptr()
    assert buf.get_data().numel() == 24 and abs(buf.usage() - 24 / 64) < 1e-9
    import pytest
    with pytest.raises(AssertionError):
        buf.get((41,))
    buf.reset()
    assert not buf.is_in_use()
    ring = RingMemBuffer("ckpt", 2, 16, torch.float32, device="cpu")
    first, second = ring.get_next_buffer(), ring.get_next_buffer()
    assert first is not second and ring.get_next_buffer() is first
    first.get((4,))
    ring.get_next_buffer()
    with pytest.raises(AssertionError):
        ring.get_next_buffer()      # back at `first`, which is still in use
    text, vals = report_memory("stage 0", get_list=True)
    assert text.startswith("stage 0 memory (MB) | allocated:") and len(vals) == 4
    big = torch.zeros(1 << 18)
    rows = debug_mem_report(min_mb=0.5)
    assert any(r[1] == (1 << 18,) and r[3] >= 1.0 for r in rows)
    del big


def test_plan_validation_messages():
    import copy
    import pytest
    from superscaler_b200.runtime.trainer import Trainer
    from helpers import tiny_gpt_plan
    good = tiny_gpt_plan()
    bad = copy.deepcopy(good)
    bad["micro_batch_size"] = 3
    with pytest.raises(ValueError, match="does not divide the global batch"):
        Trainer(bad, device="cpu")
    bad = copy.deepcopy(good)
    bad["model_parallel_size_of_each_op"][0][4] = 2
    with pytest.raises(ValueError, match="stage 0 op 4: tp 2 x dp 1"):
        Trainer(bad, device="cpu")
    bad = copy.deepcopy(good)
    bad["recompute_ops"][0].pop()
    with pytest.raises(ValueError, match="recompute_ops has"):
        Trainer(bad, device="cpu")
    from helpers import tiny_t5_plan
    bad = tiny_t5_plan(num_gpus=(2,), tp=[2])
    bad["model_parallel_size_of_each_op"][0][5], bad["data_parallel_size_of_each_op"][0][5] = 1, 2
    with pytest.raises(ValueError, match="a T5 stage keeps one"):
        Trainer(bad, device="cpu", world_size=2)


def test_recompute_segment_may_end_right_after_a_projection():
    """The deferred bias of the attention output / MLP down projection (a parameter handed to the following
    dropout + add op) can be an OUTPUT of a checkpointed segment: per-op recompute flags that stop between the two
    ops must train like the plan without recompute (the parameter used to become an output node of the
    checkpoint function, and the replay recursed without end)."""
    import torch
    from superscaler_b200.data.synthetic import gpt_batch
    from superscaler_b200.runtime.trainer import Trainer
    from helpers import tiny_gpt_plan
    ov = dict(hidden_dropout=0.0, attention_dropout=0.0)

    def losses(plan):
        t = Trainer(plan, model_overrides=ov, lr_warmup_steps=0, device="cpu", lr=1e-3)
        return [t.loss_value(t.train_step(gpt_batch(4, 128, 512, seed=1))) for _ in range(3)]

    base = losses(tiny_gpt_plan())
    plan = tiny_gpt_plan()
    rc = [0] * len(plan["recompute_ops"][0])
    for i in (2, 3, 4, 5, 6, 7, 10, 11, 12, 15, 16, 17, 18, 19, 20):     # ..., dense (7) | dropout-add (8) not
        rc[i] = 1
    plan["recompute_ops"] = [rc]
    got = losses(plan)
    # not bitwise: where a segment boundary separates a LayerNorm from its residual branch, the two gradient branches
    # are added after bf16 rounding instead of inside the LayerNorm backward
    assert max(abs(a - b) for a, b in zip(got, base)) < 3e-4, (got, base)


def test_random_per_op_recompute_flags_do_not_change_training():
    """Per-op recompute fuzz (single process): any 0/1 pattern over the ops, with segments starting and ending
    anywhere, trains like the plan that keeps everything (the search sets these flags op by op)."""
    import random
    import torch
    from superscaler_b200.data import synthetic as syn
    from superscaler_b200.runtime.trainer import Trainer
    from helpers import tiny_gpt_plan, tiny_resnet_plan, tiny_t5_plan
    rng = random.Random(23)
    cases = [
        ("gpt", tiny_gpt_plan, dict(hidden_dropout=0.0, attention_dropout=0.0),
         lambda: syn.gpt_batch(4, 128, 512, seed=1), 3e-3),     # segment ends split fused op groups: rounding
        ("t5", tiny_t5_plan, dict(hidden_dropout=0.0, attention_dropout=0.0),
         lambda: syn.t5_batch(4, 64, 32, 256, seed=1), 3e-3),
        ("resnet", lambda: tiny_resnet_plan(global_bs=16, micro_bs=8), dict(image_size=64, num_classes=16),
         lambda: syn.resnet_batch(16, 64, 16, seed=1, dtype=torch.float32), 2e-2),
    ]
    for name, plan_fn, ov, batch_fn, tol in cases:
        def losses(plan):
            t = Trainer(plan, model_overrides=ov, lr_warmup_steps=0, device="cpu", lr=1e-3)
            b = batch_fn()
            return [t.loss_value(t.train_step(b)) for _ in range(2)]
        base = losses(plan_fn())
        for trial in range(4):
            plan = plan_fn()
            n = len(plan["recompute_ops"][0])
            rc, cur = [], rng.randint(0, 1)
            while len(rc) < n:
                rc += [cur] * rng.randint(1, 6)
                cur = 1 - cur
            rc = rc[:n]
            # the ops the search never recomputes (embeddings, the loss op; reference: search/model_ops_info.py:76-90)
            never = {"encoder-embedding", "decoder-embedding", "gpt-post-process", "t5-post-process", "final-layernorm",
                     "fc", "conv1"}
            names = Trainer(plan_fn(), model_overrides=ov, device="cpu").op_names
            rc = [0 if names[i] in never else rc[i] for i in range(n)]
            plan["recompute_ops"] = [rc]
            got = losses(plan)
            assert max(abs(a - b) for a, b in zip(got, base)) < tol, (name, trial, got, base, rc)


def test_peer_memory_groups_must_sit_on_one_node(monkeypatch):
    """Rank sets that cross a node boundary (LOCAL_WORLD_SIZE consecutive ranks per node) cannot use the peer-memory
    kernels; without the launcher's variable the whole job counts as one node."""
    from superscaler_b200.parallel.state import ParallelState
    ps = ParallelState([8, 8], rank=5, world_size=16)
    monkeypatch.delenv("LOCAL_WORLD_SIZE", raising=False)
    assert ps.same_node(range(16))
    monkeypatch.setenv("LOCAL_WORLD_SIZE", "8")
    assert ps.same_node((0, 1, 2, 3)) and ps.same_node(range(8, 16)) and ps.same_node((12,))
    assert not ps.same_node((6, 7, 8, 9)) and not ps.same_node((0, 8))
    monkeypatch.setenv("LOCAL_WORLD_SIZE", "4")
    assert not ps.same_node(range(8)) and ps.same_node((4, 5, 6, 7))


def test_masked_lm_loss_is_mean_over_unmasked_tokens():
    """The loss of a batch with a loss mask is the mean cross entropy of the unmasked tokens only, and so are its
    gradients (reference: runtime/pretrain_gpt.py:64-72)."""
    from superscaler_b200.ops import functional as F
    torch.manual_seed(3)
    tokens, hidden, vocab = 24, 16, 40
    x = torch.randn(tokens, hidden, requires_grad=True)
    w = torch.randn(vocab, hidden, requires_grad=True)
    labels = torch.randint(0, vocab, (tokens,))
    mask = (torch.rand(tokens) < 0.4).float()
    mask[0] = 1.0
    weights = mask / mask.sum().clamp(min=1.0)
    loss = F.lm_head_cross_entropy(x, w, labels, weights, 0, 1.0, None)
    loss.backward()
    x2, w2 = x.detach().clone().requires_grad_(), w.detach().clone().requires_grad_()
    keep = mask.bool()
    ref = torch.nn.functional.cross_entropy((x2 @ w2.t())[keep], labels[keep])
    ref.backward()
    # the CPU restatement of the GEMM rounds its result like the bf16 kernel does
    assert abs(loss.item() - ref.item()) < 2e-2
    assert torch.allclose(x.grad, x2.grad, atol=2e-2) and torch.allclose(w.grad, w2.grad, atol=2e-2)
    unmasked = torch.nn.functional.cross_entropy(x2 @ w2.t(), labels)
    assert abs(loss.item() - unmasked.item()) > 5e-2          # and it is not the mean over all tokens

    # through the trainer: a half-masked batch reports the mean over its unmasked half, not half of it
    plan = tiny_gpt_plan(global_bs=2, micro_bs=2)
    t = Trainer(plan, model_overrides=NODROP, lr_warmup_steps=0, device="cpu")
    batch = gpt_batch(2, plan["seq_length"], 512, seed=1)
    full = t.evaluate([dict(batch)])["lm loss"]
    batch["loss_mask"] = torch.ones_like(batch["labels"], dtype=torch.float32)
    ones = t.evaluate([dict(batch)])["lm loss"]
    batch["loss_mask"][:, ::2] = 0.0
    half = t.evaluate([dict(batch)])["lm loss"]
    assert abs(full - ones) < 1e-4
    assert abs(half - ones) < 0.5 and half > 0.7 * ones


def test_a_step_with_non_finite_gradients_is_skipped_and_counted():
    import torch
    from superscaler_b200.runtime.trainer import Trainer
    from helpers import tiny_gpt_plan
    t = Trainer(tiny_gpt_plan(), device="cpu", lr_warmup_steps=0)
    before = t.store.master.clone()
    t.store.grad.fill_(1.0)
    t.store.grad[3] = float("inf")
    t.optimizer.step(lr=1e-3)
    assert torch.equal(t.store.master, before) and t.optimizer.skipped_steps() == 1
    assert float(t.store.grad.abs().sum()) == 0.0                       # the bad gradients do not leak into the next step
    t.store.grad.fill_(1.0)
    t.optimizer.step(lr=1e-3)
    assert not torch.equal(t.store.master, before) and t.optimizer.skipped_steps() == 1
