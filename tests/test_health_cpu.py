"""Failure detection without any GPU fault: host-side heartbeat / failure store, a rank that raises in a gloo job,
a dropped flag in the model of the kernels' epoch-flag protocol, a corrupted checkpoint shard."""
import os

import pytest
import torch
import torch.distributed as dist

from dist_utils import run_ranks
from helpers import tiny_gpt_plan
from superscaler_b200.parallel import flag_protocol as fp
from superscaler_b200.runtime import checkpointing
from superscaler_b200.runtime.health import DictStore, HealthMonitor, PeerFailure


def test_monitor_reports_published_failure_and_stale_heartbeat():
    store, now = DictStore(), [0.0]
    a = HealthMonitor(store, 0, 2, stale_after_s=10, clock=lambda: now[0])
    b = HealthMonitor(store, 1, 2, stale_after_s=10, clock=lambda: now[0])
    a.beat(0)
    b.beat(0)
    now[0] = 5.0
    b.beat(1)
    a.beat(1)                       # peer made progress: fine
    now[0] = 30.0
    with pytest.raises(PeerFailure, match="stuck at step 1"):
        a.beat(2)                   # rank 1 silent for 25 s
    with pytest.raises(ValueError):
        with b.guard():
            raise ValueError("boom")
    with pytest.raises(PeerFailure, match="ValueError: boom") as e:
        a.check_peers()
    assert e.value.rank == 1


def test_monitor_reports_rank_that_never_joins():
    store, now = DictStore(), [0.0]
    a = HealthMonitor(store, 0, 2, stale_after_s=10, clock=lambda: now[0])
    a.beat(0)
    now[0] = 11.0
    with pytest.raises(PeerFailure, match="never published"):
        a.beat(1)


def _failing_job(rank, world, fail_rank):
    store = dist.distributed_c10d._get_default_store()
    mon = HealthMonitor(store, rank, world, stale_after_s=30)
    x = torch.ones(4)
    seen = None
    try:
        for step in range(6):
            mon.beat(step)                       # before the collective of this step
            with mon.guard():
                if rank == fail_rank and step == 2:
                    raise RuntimeError("injected failure")
                # the failing rank leaves between steps; the others must not enter the next collective with it
                if step < 2:
                    dist.all_reduce(x)
                else:
                    import time
                    time.sleep(0.3)              # give the failure time to be published
    except PeerFailure as e:
        seen = (e.rank, e.reason)
    except RuntimeError as e:
        assert rank == fail_rank and "injected" in str(e)
        seen = "self"
    assert seen == "self" if rank == fail_rank else (seen is not None and seen[0] == fail_rank and "injected" in seen[1]), seen


def test_survivors_learn_of_a_failed_rank_before_the_next_collective():
    run_ranks(_failing_job, 3, 1, timeout=120)


def test_dropped_flag_times_out_and_later_epochs_recover():
    lost = {(1, 0, 0, 3)}          # rank 0's arrival at rank 1 is lost in epoch 3
    board = fp.FlagBoard(drop=lambda o, s, p, e: (o, s, p, e) in lost)
    assert fp.barrier(board, 2, 0, 1) == {0: fp.OK, 1: fp.OK}
    st = fp.barrier(board, 2, 0, 3, limit=50)
    assert st == {0: fp.OK, 1: fp.PEER_TIMEOUT}
    # a stale flag (epoch 1) never satisfied the wait for epoch 3, and epoch 5 works again
    assert fp.barrier(board, 2, 0, 5) == {0: fp.OK, 1: fp.OK}
    # a late flag of an old epoch is harmless
    board.post(1, 0, 0, 3)
    assert board.flags[(1, 0, 0)] == 5


def test_corrupted_checkpoint_shard_is_reported(tmp_path):
    from superscaler_b200.runtime.trainer import Trainer
    t = Trainer(tiny_gpt_plan(), model_overrides=dict(hidden_dropout=0.0, attention_dropout=0.0), lr_warmup_steps=0,
                device="cpu")
    path = checkpointing.save_checkpoint(t, str(tmp_path))
    with open(path, "r+b") as f:
        f.truncate(os.path.getsize(path) // 2)
    with pytest.raises(checkpointing.CheckpointError, match="model_optim_rng.pt"):
        checkpointing.load_checkpoint(t, str(tmp_path))


def _cli_rank(rank, world, port, plan_path, inject):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    import torch
    torch.set_num_threads(1)
    from superscaler_b200.runtime import pretrain
    pretrain.main(["--flexpipe-config", plan_path, "--train-iters", "6", "--lr-decay-iters", "10", "--hidden-dropout",
                   "0", "--attention-dropout", "0", "--distributed-backend", "gloo", "--health-check",
                   "--inject-failure", inject])


def test_training_cli_stops_instead_of_hanging_when_a_rank_fails(tmp_path):
    """Host-side fault injection through the training entry point: rank 1 raises at iteration 2 of a dp-2 run.
    Neither process may hang: the failing rank exits with its exception, the survivor leaves either at its next
    heartbeat check (exit code 3) or with the error of the collective that lost its peer."""
    import json
    import torch.multiprocessing as mp
    from dist_utils import _free_port
    plan_path = tmp_path / "gpt_tiny_dp2.json"
    plan_path.write_text(json.dumps(tiny_gpt_plan(num_gpus=(2,), tp=[1])))
    ctx = mp.get_context("spawn")
    port = _free_port()
    procs = [ctx.Process(target=_cli_rank, args=(r, 2, port, str(plan_path), "1:2")) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
    alive = [p for p in procs if p.is_alive()]
    for p in alive:
        p.terminate()
    assert not alive, "a rank hung after its peer failed"
    assert procs[1].exitcode not in (0, None)
    assert procs[0].exitcode not in (0, None)


def _cli_train(rank, world, port, argv):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    import torch
    torch.set_num_threads(1)
    from superscaler_b200.runtime import pretrain
    pretrain.main(argv)


def test_restart_on_fewer_ranks_from_a_checkpoint_of_another_plan(tmp_path, capsys):
    """Elastic recovery by restart: a tensor-parallel run on two ranks saves a checkpoint; the job continues on ONE
    rank under a one-rank plan, with the shards merged and re-sliced, at the iteration and loss level it had."""
    import json
    import re
    import torch.multiprocessing as mp
    from dist_utils import _free_port
    from superscaler_b200.runtime import pretrain
    common = ["--lr-decay-iters", "100", "--hidden-dropout", "0", "--attention-dropout", "0", "--lr", "1e-3",
              "--lr-warmup-fraction", "0"]
    two = tmp_path / "gpt_tiny_tp2.json"
    two.write_text(json.dumps(tiny_gpt_plan(num_gpus=(2,), tp=[2])))
    one = tmp_path / "gpt_tiny_1.json"
    one.write_text(json.dumps(tiny_gpt_plan()))
    ckpt = str(tmp_path / "ckpt")
    ctx = mp.get_context("spawn")
    port = _free_port()
    argv = ["--flexpipe-config", str(two), "--train-iters", "4", "--distributed-backend", "gloo", "--save", ckpt] + common
    procs = [ctx.Process(target=_cli_train, args=(r, 2, port, argv)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(180)
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    # reference: the same six iterations on one rank from scratch (same seed, same batches)
    pretrain.main(["--flexpipe-config", str(one), "--train-iters", "6"] + common)
    scratch = [float(x) for x in re.findall(r"lm loss: ([0-9.E+-]+)", capsys.readouterr().out)]
    pretrain.main(["--flexpipe-config", str(one), "--train-iters", "6", "--load", ckpt, "--load-resharded"] + common)
    out = capsys.readouterr().out
    resumed = [float(x) for x in re.findall(r"lm loss: ([0-9.E+-]+)", out)]
    assert "iteration        5/       6" in out and "iteration        4/" not in out and len(resumed) == 2
    # weights carried over: the resumed run is where the uninterrupted one was, not back at the initial loss
    # (optimizer moments restart, so the match is close, not exact)
    assert abs(resumed[0] - scratch[4]) < 0.05 * scratch[4] and resumed[0] < scratch[0] - 0.1


def _cli_train_logged(rank, world, port, argv, log):
    import contextlib
    with open(f"{log}.{rank}", "w") as f, contextlib.redirect_stdout(f):
        _cli_train(rank, world, port, argv)


def test_interleaved_cli_run_resumes_exactly(tmp_path):
    """`--interleave-factor 2` on two pipeline ranks: a run stopped after 2 of 4 iterations and resumed from its
    checkpoint (weights of both chunks, optimizer state, schedule) prints the losses of the uninterrupted run."""
    import json
    import re
    import torch.multiprocessing as mp
    from dist_utils import _free_port
    plan = tmp_path / "gpt_tiny_pp2.json"
    plan.write_text(json.dumps(tiny_gpt_plan(num_gpus=(1, 1), micro_bs=1)))
    common = ["--flexpipe-config", str(plan), "--distributed-backend", "gloo", "--interleave-factor", "2",
              "--lr-decay-iters", "100", "--lr", "1e-3", "--lr-warmup-fraction", "0", "--hidden-dropout", "0",
              "--attention-dropout", "0"]
    ctx = mp.get_context("spawn")

    def launch(name, extra):
        port = _free_port()
        log = str(tmp_path / name)
        procs = [ctx.Process(target=_cli_train_logged, args=(r, 2, port, common + extra, log)) for r in range(2)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(180)
        assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
        text = open(log + ".0").read() + open(log + ".1").read()
        return [float(x) for x in re.findall(r"lm loss: ([0-9.E+-]+)", text)]

    whole = launch("whole", ["--train-iters", "4"])
    ckpt = str(tmp_path / "ckpt")
    first = launch("first", ["--train-iters", "2", "--save", ckpt])
    second = launch("second", ["--train-iters", "4", "--load", ckpt])
    assert len(whole) == 4 and first == whole[:2] and len(second) == 2
    assert max(abs(a - b) for a, b in zip(second, whole[2:])) < 1e-4, (second, whole)


def test_device_status_word_stops_training_and_saving(tmp_path):
    """A kernel that gave up a bounded wait leaves a status word behind; the trainer reads it where the host
    synchronises anyway (loss read-back, checkpoint save), raises, and tells the other ranks through the monitor."""
    import pytest
    from helpers import tiny_gpt_plan
    from superscaler_b200.data.synthetic import gpt_batch
    from superscaler_b200.runtime import checkpointing
    from superscaler_b200.runtime.health import DeviceStatusError, DictStore, HealthMonitor, PeerFailure
    from superscaler_b200.runtime.trainer import Trainer
    plan = tiny_gpt_plan()
    t = Trainer(plan, lr_warmup_steps=0, device="cpu",
                model_overrides=dict(hidden_dropout=0.0, attention_dropout=0.0, max_tp=1))
    stats = t.train_step(gpt_batch(plan["global_batch_size"], plan["seq_length"], 512, seed=1))
    assert t.loss_value(stats) > 0                       # status 0: nothing happens
    store = DictStore()
    t.health_monitor = HealthMonitor(store, rank=0, world=2)
    codes = iter([2, 2])
    t._read_device_status = lambda: next(codes, 0)       # what a timed-out peer wait would leave in the status word
    with pytest.raises(DeviceStatusError) as e:
        t.loss_value(stats)
    assert e.value.code == 2 and "peer" in str(e.value)
    with pytest.raises(DeviceStatusError):
        checkpointing.save_checkpoint(t, str(tmp_path))
    assert not any(tmp_path.iterdir())                   # nothing was written
    with pytest.raises(PeerFailure):                     # the other rank learns of it before its next collective
        HealthMonitor(store, rank=1, world=2).check_peers()
    checkpointing.save_checkpoint(t, str(tmp_path))      # status read and cleared: saving works again
    assert any(tmp_path.iterdir())


def test_guard_words_report_the_first_overwritten_word_and_stop_training():
    """Guard bands around a buffer (what SSB_CANARIES=1 puts around symmetric memory): intact after in-range writes,
    a write one element past either end is reported with its position, and the trainer refuses to go on."""
    import torch
    from superscaler_b200.data.synthetic import gpt_batch
    from superscaler_b200.parallel import guards
    from superscaler_b200.runtime.health import DeviceStatusError
    from superscaler_b200.runtime.trainer import Trainer
    from helpers import tiny_gpt_plan
    for dtype, n in ((torch.float32, 1000), (torch.bfloat16, 1001), (torch.int32, 7)):
        b = guards.GuardedBuffer(n, dtype, "cpu", name="payload")
        assert b.body.numel() == n and b.body_offset_bytes == guards.GUARD_BYTES
        assert b.raw.data_ptr() + b.body_offset_bytes == b.body.data_ptr()
        b.body.fill_(3)
        assert b.check() == []
        b.raw[b.guard_elems + n + b.tail_pad_elems] = 1                    # first element behind the payload
        (line,) = b.check()
        assert "guard word 0 behind the payload" in line
        b.arm()
        b.raw[b.guard_elems - 1] = 1                                       # last element in front of it
        (line,) = b.check()
        assert "in front of the payload" in line and f"guard word {guards.GUARD_BYTES // 4 - 1}" in line
    reg = guards.REGISTRY
    saved = list(reg.buffers)
    try:
        reg.buffers.clear()
        t = Trainer(tiny_gpt_plan(), device="cpu", lr_warmup_steps=0,
                    model_overrides=dict(hidden_dropout=0.0, attention_dropout=0.0))
        buf = reg.add(guards.GuardedBuffer(64, torch.float32, "cpu", name="symmetric buffer of 64"))
        stats = t.train_step(gpt_batch(4, 128, 512, seed=1))
        t.loss_value(stats)                                                # guards intact: nothing happens
        buf.raw[0] = 0.0
        with pytest.raises(DeviceStatusError, match="guard word 0 in front of the payload"):
            t.loss_value(stats)
    finally:
        reg.buffers[:] = saved
