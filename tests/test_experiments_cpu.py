"""The experiment driver: the commands it issues for each mode, and tables / figures from runtime CSVs."""
import os

from superscaler_b200 import experiments as E


def test_modes_issue_the_expected_commands(tmp_path, capsys):
    E.main(["search", "--model", "gpt", "--mode", "small", "--results", str(tmp_path), "--dry-run"])
    out = capsys.readouterr().out
    assert "superscaler_b200.search.search" in out and "--model-size 1_3B" in out and "--num-gpus-per-node 4" in out
    assert "--global-batch-size 512" in out and "--micro-batch-size 1 2 4 8" in out
    E.main(["baseline", "--model", "resnet", "--mode", "large", "--results", str(tmp_path), "--max-gpus", "8", "--dry-run"])
    out = capsys.readouterr().out
    assert out.count("superscaler_b200.search.grid_plan") == 3                 # 500M / 2B / 4B fit into 8 GPUs
    assert "--global-batch-size 1536" in out and "--micro-batch-size 16 32 48 64" in out
    E.main(["search", "--model", "gpt", "--mode", "scale", "--results", str(tmp_path), "--dry-run"])
    out = capsys.readouterr().out
    assert out.count("--num-layers") == 8 and "--num-layers 1024" in out and "--num-gpus-per-node 8" in out
    # execute: one launch per saved plan
    cfg = tmp_path / "aceso" / "configs" / "gpt" / "1_3B" / "top_configs"
    (cfg / "gpt_1_3B_2stages_x.json").write_text("{}")
    E.main(["execute", "--model", "gpt", "--mode", "small", "--results", str(tmp_path), "--dry-run"])
    out = capsys.readouterr().out
    assert "--nproc-per-node=4" in out and "superscaler_b200.runtime.pretrain" in out and "--train-iters 3" in out


def test_collect_and_plot(tmp_path, capsys):
    header = "global_batch_size,time,forward-backward,backward-params-all-reduce,optimizer,max_allocated_memory(MB)\n"
    for system, t in (("grid", 2000.0), ("aceso", 1600.0)):
        run = tmp_path / system / "runtime" / "gpt" / "1_3B" / "csv"
        os.makedirs(run)
        for r in range(2):
            (run / f"gpt_1_3B_2stages_x_stage{r}_rank{r}.csv").write_text(header + f"512,{t - 10 * r},1,1,1,{9000 + r}\n")
        log = tmp_path / system / "search" / "gpt" / "1_3B"
        os.makedirs(log)
        (log / "gpt_1_3B_summary_x.csv").write_text("search_cost\n12.5\n")
    pred = tmp_path / "aceso" / "configs" / "gpt" / "1_3B" / "csv"
    os.makedirs(pred)
    (pred / "info_gpt_1_3B_2stages_x.csv").write_text("stage,time,memory\n0,1500.0,8800\n1,1550.0,8700\n")
    E.main(["collect", "--mode", "small", "--results", str(tmp_path)])
    out = capsys.readouterr().out
    assert "| aceso | 320.0 |" in out and "| grid | 256.0 |" in out          # 512 / 1.6 s and 512 / 2.0 s
    assert "| aceso | 1.25 |" in out                                           # normalised to the grid planner
    assert "| predicted | 1.55 |" in out and "| actual | 1.6 |" in out
    E.main(["plot", "--mode", "small", "--results", str(tmp_path)])
    figs = [l for l in capsys.readouterr().out.splitlines() if l.endswith(".svg")]
    assert any("e2e_norm_thpt_small_gpt" in f for f in figs)
    svg = open([f for f in figs if "e2e_norm_thpt_small_gpt" in f][0]).read()
    assert svg.startswith("<svg") and "1.25" in svg and "<rect" in svg
