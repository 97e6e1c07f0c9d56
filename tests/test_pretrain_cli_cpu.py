"""The training entry point writes the per-rank CSVs, and the result-collection helpers read them."""
import json
import os

from helpers import tiny_gpt_plan
from superscaler_b200.runtime import pretrain
from superscaler_b200.utils import results


def test_pretrain_writes_csv_and_results_read_it(tmp_path):
    plan_path = tmp_path / "gpt_tiny_1stages_demo.json"
    plan_path.write_text(json.dumps(tiny_gpt_plan()))
    log = tmp_path / "logs"
    pretrain.main(["--flexpipe-config", str(plan_path), "--train-iters", "2", "--log-path", str(log),
                   "--lr-decay-iters", "10", "--hidden-dropout", "0", "--attention-dropout", "0", "--save", str(tmp_path / "ckpt")])
    csv_path = log / "csv" / "gpt_tiny_1stages_demo_stage0_rank0.csv"
    assert csv_path.is_file()
    row = results.read_runtime_csv(str(csv_path))
    assert row["global_batch_size"] == 4 and row["time"] > 0
    thpt = results.throughput(str(log), "gpt_tiny_1stages_demo")
    assert abs(thpt - 4 / (row["time"] / 1000.0)) < 1e-6
    name, best = results.best_throughput(str(log))
    assert name == "gpt_tiny_1stages_demo" and best == thpt
    assert os.path.isfile(tmp_path / "ckpt" / "latest_checkpointed_iteration.txt")
    # resume: a second run starts from iteration 2 and performs one more
    pretrain.main(["--flexpipe-config", str(plan_path), "--train-iters", "3", "--lr-decay-iters", "10", "--hidden-dropout", "0", "--attention-dropout", "0",
                   "--load", str(tmp_path / "ckpt"), "--save", str(tmp_path / "ckpt")])
    assert (tmp_path / "ckpt" / "latest_checkpointed_iteration.txt").read_text().strip() == "3"


def test_cost_model_accuracy(tmp_path):
    log = tmp_path / "logs"
    os.makedirs(log / "csv")
    for r, t in enumerate([100.0, 110.0]):
        (log / "csv" / f"cfg_stage{r}_rank{r}.csv").write_text(
            "global_batch_size,time,forward-backward,backward-params-all-reduce,optimizer,max_allocated_memory(MB)\n"
            f"8,{t},90,5,5,{1000 + r}\n")
    pred = tmp_path / "info.csv"
    pred.write_text("stage,time,memory\n0,99.0,900\n1,104.5,950\n")
    acc = results.cost_model_accuracy(str(pred), str(log), "cfg")
    assert acc["actual_time_ms"] == 110.0 and abs(acc["time_error_pct"] - 5.0) < 1e-9
    assert acc["actual_memory_mb"] == 1001
    assert abs(results.throughput(str(log), "cfg") - 8 / 0.110) < 1e-9


def test_pretrain_eval_tensorboard_finetune_and_timed_exit(tmp_path, capsys):
    plan_path = tmp_path / "gpt_tiny_1stages_demo.json"
    plan_path.write_text(json.dumps(tiny_gpt_plan()))
    common = ["--flexpipe-config", str(plan_path), "--lr-decay-iters", "10", "--hidden-dropout", "0",
              "--attention-dropout", "0"]
    pretrain.main(common + ["--train-iters", "2", "--eval-interval", "1", "--eval-iters", "1", "--tensorboard-dir",
                            str(tmp_path / "tb"), "--save", str(tmp_path / "ckpt")])
    out = capsys.readouterr().out
    assert out.count("validation loss at iteration") == 2 and "lm loss ppl value" in out
    assert any(f.startswith("events.out.tfevents") for f in os.listdir(tmp_path / "tb"))
    # --finetune loads the weights and restarts the iteration count: two more iterations run
    pretrain.main(common + ["--train-iters", "2", "--load", str(tmp_path / "ckpt"), "--finetune", "--no-load-rng"])
    out = capsys.readouterr().out
    assert "iteration        1/       2" in out and "iteration        2/       2" in out
    # a run past its time budget stops after the first iteration and still saves
    pretrain.main(common + ["--train-iters", "50", "--exit-duration-in-mins", "0", "--save", str(tmp_path / "ckpt2")])
    out = capsys.readouterr().out
    assert "exiting after" in out and "iteration        2/" not in out
    assert (tmp_path / "ckpt2" / "latest_checkpointed_iteration.txt").read_text().strip() == "1"


def test_pretrain_on_a_token_corpus(tmp_path, capsys):
    """--data-path: documents of a periodic token pattern; the model learns it within a few dozen iterations, and
    a run resumed from the checkpoint keeps the learned loss level."""
    import re
    import numpy as np
    rng = np.random.RandomState(0)
    docs = []
    for _ in range(40):
        start, n = int(rng.randint(0, 16)), int(rng.randint(100, 400))
        docs.append(((np.arange(n) + start) % 16 + 20).astype(np.uint16))
    np.concatenate(docs).tofile(tmp_path / "corpus.bin")
    np.save(tmp_path / "corpus.npy", np.asarray([len(d) for d in docs], dtype=np.int32))
    plan_path = tmp_path / "gpt_tiny_1stages_data.json"
    plan_path.write_text(json.dumps(tiny_gpt_plan(seq=64, hidden=64, heads=2, head_dim=32, vocab=64)))
    common = ["--flexpipe-config", str(plan_path), "--data-path", str(tmp_path / "corpus"), "--lr", "3e-3",
              "--lr-decay-style", "constant", "--lr-warmup-fraction", "0", "--hidden-dropout", "0",
              "--attention-dropout", "0", "--log-interval", "10"]
    pretrain.main(common + ["--train-iters", "40", "--save", str(tmp_path / "ckpt")])
    losses = [float(x) for x in re.findall(r"lm loss: ([0-9.E+-]+)", capsys.readouterr().out)]
    assert len(losses) == 4 and losses[-1] < 0.5 * losses[0]
    pretrain.main(common + ["--train-iters", "50", "--load", str(tmp_path / "ckpt"), "--eod-mask-loss", "21"])
    more = [float(x) for x in re.findall(r"lm loss: ([0-9.E+-]+)", capsys.readouterr().out)]
    assert len(more) == 1 and more[0] < losses[0]


def test_throughput_table(tmp_path, capsys):
    log = tmp_path / "logs"
    os.makedirs(log / "csv")
    for name, times in (("a_2stages_x", [100.0, 110.0]), ("b_1stages_x", [50.0])):
        for r, t in enumerate(times):
            (log / "csv" / f"{name}_stage{r}_rank{r}.csv").write_text(
                "global_batch_size,time,forward-backward,backward-params-all-reduce,optimizer,max_allocated_memory(MB)\n"
                f"8,{t},90,5,5,{1000 + r}\n")
    results.main(["--log-path", str(log), "--table"])
    out = capsys.readouterr().out.splitlines()
    assert out[2].startswith("| a_2stages_x | 2 | 110.0 | 72.73 | 1001 |")
    assert out[3].startswith("| b_1stages_x | 1 | 50.0 | 160.00 | 1000 |")


def test_synthetic_run_resumed_past_iteration_four_sees_the_same_batches(tmp_path, capsys):
    """The synthetic batch of iteration k is the same in a fresh run and in one resumed at any iteration: seven
    iterations in one go print the losses of five iterations plus two after a restart."""
    import re
    plan_path = tmp_path / "gpt_tiny_1stages_resume.json"
    plan_path.write_text(json.dumps(tiny_gpt_plan()))
    common = ["--flexpipe-config", str(plan_path), "--lr-decay-iters", "20", "--hidden-dropout", "0",
              "--attention-dropout", "0", "--lr", "1e-3"]
    pretrain.main(common + ["--train-iters", "7"])
    whole = re.findall(r"lm loss: ([0-9.E+-]+)", capsys.readouterr().out)
    pretrain.main(common + ["--train-iters", "5", "--save", str(tmp_path / "ckpt")])
    first = re.findall(r"lm loss: ([0-9.E+-]+)", capsys.readouterr().out)
    pretrain.main(common + ["--train-iters", "7", "--load", str(tmp_path / "ckpt")])
    second = re.findall(r"lm loss: ([0-9.E+-]+)", capsys.readouterr().out)
    assert len(whole) == 7 and first + second == whole


def test_t5_trains_on_span_corruption_batches_of_a_sentence_corpus(tmp_path):
    """Text -> `data.preprocess --split-sentences` -> T5Dataset (sentinels appended to the WordPiece vocabulary) ->
    the batches `runtime.pretrain --data-path --vocab-file` feeds a T5 plan."""
    import math
    import numpy as np
    import torch
    from helpers import tiny_t5_plan
    from superscaler_b200.data import preprocess
    from superscaler_b200.runtime.pretrain import make_dataset_batch_fn
    from superscaler_b200.runtime.trainer import Trainer
    words = ["[PAD]", "[UNK]", "[CLS]", "[SEP]", "[MASK]"] + [f"w{i}" for i in range(60)] + [".", "!", "?"]
    vocab = tmp_path / "vocab.txt"
    vocab.write_text("\n".join(words) + "\n")
    rs = np.random.RandomState(1)
    docs = [" ".join(" ".join(rs.choice(words[5:65], size=rs.randint(5, 10))) + "." for _ in range(rs.randint(4, 8)))
            for _ in range(10)]
    (tmp_path / "docs.txt").write_text("\n".join(docs) + "\n")
    prefix = str(tmp_path / "corpus")
    preprocess.main(["--input", str(tmp_path / "docs.txt"), "--output", prefix, "--split-sentences", "--tokenizer-type",
                     "BertWordPieceLowerCase", "--vocab-file", str(vocab)])
    plan = tiny_t5_plan(vocab=256)                          # 68 words + [BOS] [EOS] + 100 sentinels fit
    t = Trainer(plan, device="cpu", lr_warmup_steps=0, lr=2e-3,
                model_overrides=dict(hidden_dropout=0.0, attention_dropout=0.0))
    fn = make_dataset_batch_fn(t, prefix, train_iters=3, seed=7, vocab_file=str(vocab))
    b = fn(0)
    assert b["ids"].shape == (4, t.cfg.seq_length) and b["dec_ids"].shape == (4, t.cfg.dec_seq_length)
    assert (b["dec_ids"][:, 0] == 68).all()                # [BOS] is the first id appended after the vocabulary
    assert ((b["ids"] >= 70) & (b["ids"] < 170)).any()     # sentinels in the encoder input
    assert torch.equal(fn(0)["ids"], b["ids"])
    losses = [t.loss_value(t.train_step(fn(i))) for i in range(3)]
    assert all(math.isfinite(v) for v in losses)


def test_split_holds_out_validation_and_test_documents(tmp_path, capsys):
    """--split on a corpus in Megatron-LM's format: the first 30 documents (pattern A) train, the held-out parts hold
    documents of a pattern the model never saw, so their loss stays far above the training loss."""
    import re
    import numpy as np
    from superscaler_b200.data import mmap_format
    rng = np.random.RandomState(0)
    docs = []
    for d in range(40):
        n = int(rng.randint(200, 400))
        if d < 30:
            docs.append(((np.arange(n) + int(rng.randint(0, 16))) % 16 + 20).tolist())     # periodic, learnable
        else:
            docs.append(rng.randint(40, 60, size=n).tolist())                              # unseen token range
    mmap_format.write(str(tmp_path / "corpus"), docs, list(range(41)), dtype=np.uint16)
    plan_path = tmp_path / "gpt_tiny_1stages_split.json"
    plan_path.write_text(json.dumps(tiny_gpt_plan(seq=64, hidden=64, heads=2, head_dim=32, vocab=64)))
    pretrain.main(["--flexpipe-config", str(plan_path), "--data-path", str(tmp_path / "corpus"), "--lr", "3e-3",
                   "--lr-decay-style", "constant", "--lr-warmup-fraction", "0", "--hidden-dropout", "0",
                   "--attention-dropout", "0", "--log-interval", "10", "--train-iters", "40",
                   "--split", "30,6,4", "--eval-interval", "20", "--eval-iters", "1"])
    out = capsys.readouterr().out
    train = [float(x) for x in re.findall(r"lm loss: ([0-9.E+-]+)", out)]
    valid = [float(x) for x in re.findall(r"validation loss at iteration \d+ \| lm loss value: ([0-9.E+-]+)", out)]
    test = [float(x) for x in re.findall(r"test loss at the end of training \| lm loss value: ([0-9.E+-]+)", out)]
    assert len(valid) == 2 and len(test) == 1
    assert train[-1] < 1.5 and min(valid + test) > 2.5


def test_blend_of_two_corpora_draws_from_both_by_weight(tmp_path):
    """--data-path W1 P1 W2 P2: samples of the two corpora (told apart by their token ranges) arrive in the ratio
    of the weights."""
    import numpy as np
    from superscaler_b200.runtime.trainer import Trainer
    rng = np.random.RandomState(1)
    for name, lo in (("a", 10), ("b", 40)):
        docs = [rng.randint(lo, lo + 10, size=int(rng.randint(150, 300))).astype(np.uint16) for _ in range(12)]
        np.concatenate(docs).tofile(tmp_path / f"{name}.bin")
        np.save(tmp_path / f"{name}.npy", np.asarray([len(d) for d in docs], dtype=np.int32))
    t = Trainer(tiny_gpt_plan(seq=32, hidden=64, heads=2, head_dim=32, vocab=64), device="cpu")
    fn = pretrain.make_dataset_batch_fn(t, ["3", str(tmp_path / "a"), "1", str(tmp_path / "b")], train_iters=8, seed=5,
                                        split="9,1,0", eval_samples=8)
    gbs = t.plan["global_batch_size"]
    rows = np.concatenate([fn(i)["ids"].numpy() for i in range(8)])
    from_a = (rows < 30).all(axis=1)
    from_b = (rows >= 30).all(axis=1)
    assert (from_a | from_b).all()                       # no sample mixes the corpora
    assert abs(from_a.mean() - 0.75) < 0.05
    assert fn.valid is not None and fn.test is None
    assert fn.valid(0)["ids"].shape == (gbs, 32)
    again = pretrain.make_dataset_batch_fn(t, ["3", str(tmp_path / "a"), "1", str(tmp_path / "b")], train_iters=8, seed=5,
                                           split="9,1,0", eval_samples=8)
    assert np.array_equal(again(3)["ids"].numpy(), fn(3)["ids"].numpy())


def test_optimizer_flags_and_the_extra_columns_of_the_iteration_line(tmp_path, capsys):
    import re
    import torch
    from superscaler_b200.runtime.trainer import Trainer
    plan = tiny_gpt_plan()
    plan_path = tmp_path / "gpt_tiny_1stages_flags.json"
    plan_path.write_text(json.dumps(plan))
    pretrain.main(["--flexpipe-config", str(plan_path), "--train-iters", "3", "--lr", "1e-2", "--lr-warmup-iters", "2",
                   "--lr-decay-style", "constant", "--adam-beta1", "0.8", "--adam-beta2", "0.95", "--adam-eps", "1e-6",
                   "--init-method-std", "0.05", "--log-params-norm", "--log-num-zeros-in-grad",
                   "--hidden-dropout", "0", "--attention-dropout", "0"])
    out = capsys.readouterr().out
    lrs = [float(x) for x in re.findall(r"learning rate: ([0-9.E+-]+)", out)]
    assert lrs == [0.0, 5e-3, 1e-2]                                   # two warm-up iterations, then the full rate
    norms = [float(x) for x in re.findall(r"params norm: ([0-9.]+)", out)]
    zeros = [int(x) for x in re.findall(r"num zeros: (\d+)", out)]
    assert len(norms) == 3 and len(zeros) == 3
    t = Trainer(plan, device="cpu", model_overrides=dict(init_std=0.05), adam_betas=(0.8, 0.95), adam_eps=1e-6)
    assert t.optimizer.betas == (0.8, 0.95) and t.optimizer.eps == 1e-6
    want = float(torch.sqrt(sum(p.detach().float().pow(2).sum() for p in t.store.params.values())))
    assert abs(t.optimizer.params_norm() - want) < 1e-3 * want
    assert abs(norms[0] - want) < 2e-2 * want                          # same seed, same initialisation; no step at lr 0
    wide = Trainer(plan, device="cpu")
    assert t.optimizer.params_norm() > 1.3 * wide.optimizer.params_norm()      # std 0.05 against 0.02 (LayerNorm gains stay 1)
    assert min(zeros) > 0
    # the count is over the parameters' own entries (no alignment padding), each parameter once
    t.store.grad.fill_(1.0)
    assert t.optimizer.count_zeros_in_grad() == 0
    name = next(iter(t.store.offsets))
    off, n = t.store.offsets[name]
    t.store.grad[off:off + n] = 0.0
    assert t.optimizer.count_zeros_in_grad() == n


def test_sigterm_ends_the_run_after_an_iteration_with_a_checkpoint(tmp_path):
    """--exit-signal-handler in a child process: the signal arrives in the middle of training, the run saves and
    leaves with exit code 0, and a second run continues from that checkpoint."""
    import signal
    import subprocess
    import sys
    import time
    plan_path = tmp_path / "gpt_tiny_1stages_term.json"
    plan_path.write_text(json.dumps(tiny_gpt_plan()))
    cmd = [sys.executable, "-u", "-m", "superscaler_b200.runtime.pretrain", "--flexpipe-config", str(plan_path),
           "--train-iters", "100000", "--save", str(tmp_path / "ckpt"), "--exit-signal-handler", "--log-interval", "1",
           "--hidden-dropout", "0", "--attention-dropout", "0"]
    env = dict(os.environ, PYTHONPATH=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    p = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env)
    lines = []
    try:
        deadline = time.time() + 120
        while time.time() < deadline:
            line = p.stdout.readline()
            lines.append(line)
            assert line or p.poll() is None, "the run ended early:\n" + "".join(lines)
            if " iteration        3/" in line:          # the handler is installed long before the third iteration
                break
        else:
            raise AssertionError("no third iteration within two minutes:\\n" + "".join(lines))
        p.send_signal(signal.SIGTERM)
        rest, _ = p.communicate(timeout=120)
    finally:
        if p.poll() is None:
            p.kill()
    assert p.returncode == 0, rest
    assert "termination requested: stopping after iteration" in rest
    done = int((tmp_path / "ckpt" / "latest_checkpointed_iteration.txt").read_text())
    assert 3 <= done < 100000


def test_debug_dump_writes_op_outputs_and_gradient_statistics(tmp_path):
    from superscaler_b200.runtime import stage
    plan_path = tmp_path / "gpt_tiny_1stages_dump.json"
    plan_path.write_text(json.dumps(tiny_gpt_plan()))
    logs = str(tmp_path / "logs") + os.sep
    pretrain.main(["--flexpipe-config", str(plan_path), "--train-iters", "2", "--log-path", logs, "--debug-dump", "all",
                   "--hidden-dropout", "0", "--attention-dropout", "0"])
    assert stage.AFTER_OP_HOOKS == []                                  # the hook is gone after the run
    out = open(logs + "gpt_tiny_1stages_dump_debug_output_rank_0.log").read().splitlines()
    grad = open(logs + "gpt_tiny_1stages_dump_debug_grad_rank_0.log").read().splitlines()
    assert all(line.startswith("it 0 |") for line in out)             # the first iteration only
    names = [line.split("|")[1].split()[2] for line in out]
    assert names[0] == "encoder-embedding" and "gpt-post-process" in names and "enc-attention-qkv" in names
    assert any("| loss () |" in line for line in out)
    assert grad[0].startswith("=== iteration 0, before the reduction")
    rows = [line for line in grad if line.startswith("it 0 |")]
    assert len(rows) % 2 == 0 and any("word_embeddings.weight" in r for r in rows)
    norms = [float(r.rsplit("grad norm", 1)[1]) for r in rows]
    assert max(norms) > 0.0
