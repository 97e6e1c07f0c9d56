"""Search arguments and the mutable state shared by the policy, the primitives and the driver.

The reference keeps this state in module globals initialised at import time from sys.argv
(search/aceso_utils.py:455-531, search/aceso_policy.py:10-12, search/aceso_prims.py:10,52-54); here it is
one object, so several searches can run in one process and tests can build it directly.
"""
from __future__ import annotations

import argparse
import datetime
import json
import os
import random
import time
from dataclasses import dataclass
from typing import Dict, List, Optional

from .config import BERT_SIZES, GPT_SIZES, RESNET_SIZES, STATE_MULTIPLIERS, T5_SIZES, VIT_SIZES
from .cost_model import CostModel, CostOptions
from .database import ProfileDB
from .opinfo import expand_op_list, never_recompute_ops, read_unique_ops, tunable_ops


@dataclass
class SearchArgs:
    model_name: str = "gpt"
    model_size: str = "1_3B"
    num_layers: Optional[int] = None
    global_batch_size: int = 512
    micro_batch_size: Optional[List[int]] = None
    max_tp: Optional[int] = None
    num_nodes: int = 1
    num_gpus_per_node: int = 4
    memory_limit: int = 28000
    log_path: Optional[str] = None
    profiled_time_path: str = ""
    config_save_path: Optional[str] = None
    config_suffix: Optional[str] = None
    max_num_hops: int = 7
    max_num_trials: int = 100
    time_budget_per_trial: Optional[float] = None
    time_budget_total: float = 10
    explored_budget: Optional[int] = None    # deterministic budget: stop after this many explored plans
    start_num_stages: Optional[int] = None
    end_num_stages: Optional[int] = None
    op_group_size: int = 1
    max_op_move_steps: int = 5
    memory_pred_type: str = "MAX"
    initial_point: str = "balance"
    high_memory_rate: float = 0.9
    print_debug_info: bool = False
    consider_shared_space: bool = True
    consider_reserved_space: bool = True
    predict_delta_time: bool = False
    flex_recompute: bool = True
    add_action_tp_dp_exchange: bool = False
    peak_mem_in_backward: int = 0
    finetune_after_trial: int = 0
    multi_process: bool = True
    random_order_actions: bool = False
    support_comm_predict: bool = False
    sort_metric: str = "max_stage_time"
    finetune_tp_dp_after_trial: bool = False
    init_dim: str = "tp"
    num_partners_in_op_mig: int = 1
    continue_when_fail: bool = True
    adaptive_hyper_parameters: int = 5
    num_of_saved_configs: int = 1
    simple_prim_mbs: bool = False
    simple_prim_mig: bool = False
    only_top_1_target: bool = False
    consider_collective_memory: bool = False
    price_overlap: bool = True
    shapes: str = "reference"
    save_to_csv: Optional[str] = None
    # derived
    num_gpus: int = 0
    num_algos: int = 2
    resharding: bool = True

    def finalize(self) -> "SearchArgs":
        self.num_gpus = self.num_gpus_per_node * self.num_nodes
        if os.path.exists(self.initial_point):
            with open(self.initial_point) as f:
                d = json.load(f)
            self.model_name, self.model_size = d["model_name"], d["model_size"]
        if self.model_name not in ("resnet", "gpt", "t5", "scale-layer", "bert", "vit"):
            raise RuntimeError(f"model {self.model_name} is not supported yet.")
        if self.num_layers is None:
            if self.model_name == "resnet":
                self.num_layers = sum(RESNET_SIZES[self.model_size][0])
            elif self.model_name == "gpt":
                self.num_layers = GPT_SIZES[self.model_size][0]
            elif self.model_name == "t5":
                self.num_layers = T5_SIZES[self.model_size][0]
            elif self.model_name == "bert":
                self.num_layers = BERT_SIZES[self.model_size][0]
            elif self.model_name == "vit":
                self.num_layers = VIT_SIZES[self.model_size][0]
            else:
                raise RuntimeError("should provide --num-layers for scale-layer exp")
        if self.micro_batch_size is None:
            self.micro_batch_size = [16, 32, 48, 64] if self.model_name == "resnet" else [1, 2, 4, 8]
        # a micro-batch size that does not divide the global batch would be priced for fewer samples than the batch
        # holds (the number of micro-batches is an integer division); such candidates are dropped
        bad = [m for m in self.micro_batch_size if self.global_batch_size % m]
        if bad:
            print(f"micro-batch sizes {bad} do not divide the global batch {self.global_batch_size}: ignored")
            self.micro_batch_size = [m for m in self.micro_batch_size if m not in bad]
            assert self.micro_batch_size, "no micro-batch size divides the global batch"
        if self.start_num_stages is None or self.end_num_stages is None:
            self.start_num_stages, self.end_num_stages = 1, min(self.num_gpus, 16)
        if self.max_tp is None:
            self.max_tp = self.num_gpus_per_node
        if self.time_budget_per_trial is None:
            self.time_budget_per_trial = self.time_budget_total
        self.num_algos = 1 if self.model_name == "t5" else 2
        self.resharding = self.model_name != "t5"
        if self.config_suffix is None:
            t = datetime.datetime.now()
            self.config_suffix = f"{t.year}-{t.month}-{t.day}-{t.hour}-{t.minute}-{t.second}"
        return self


def add_cli_arguments(p: argparse.ArgumentParser) -> None:
    """The reference's flag surface (search/aceso_utils.py:359-451) plus --explored-budget / --no-price-overlap."""
    a = p.add_argument
    a("--model-name", type=str, default=None)
    a("--model-size", type=str, default=None)
    a("--num-layers", type=int, default=None)
    a("--global-batch-size", type=int, default=None)
    a("--micro-batch-size", nargs="+", type=int, default=None)
    a("--max-tp", type=int, default=None)
    a("--num-nodes", type=int, default=None)
    a("--num-gpus-per-node", type=int, default=None)
    a("--memory-limit", type=int, default=28000)
    a("--log-path", type=str, default=None)
    a("--profiled-time-path", type=str, default=None)
    a("--config-save-path", type=str, default=None)
    a("--config-suffix", type=str, default=None)
    a("--max-num-hops", type=int, default=None)
    a("--max-num-trials", type=int, default=100)
    a("--time-budget-per-trial", type=int, default=None)
    a("--time-budget-total", type=int, default=10)
    a("--explored-budget", type=int, default=None)
    a("--start-num-stages", type=int, default=None)
    a("--end-num-stages", type=int, default=None)
    a("--op-group-size", type=int, default=1)
    a("--max-op-move-steps", type=int, default=5)
    a("--memory-pred-type", type=str, default="MAX")
    a("--initial-point", type=str, default="balance",
      help="balance | imbalance_gpu | imbalance_op (the reference's), grid (best uniform plan of the stage count), "
           "both (balance and grid, the faster result is kept), or the path of a plan JSON")
    a("--high-memory-rate", type=float, default=0.9)
    a("--print-debug-info", action="store_true")
    a("--do-not-consider-shared-tensor-space", action="store_false", dest="consider_shared_space")
    a("--do-not-consider-reserved-space", action="store_false", dest="consider_reserved_space")
    a("--predict-delta-time", action="store_true")
    a("--do-not-use-flex-recompute", action="store_false", dest="flex_recompute")
    a("--add-action-tp-dp-exchange", action="store_true")
    a("--peak-mem-in-backward", type=int, default=0)
    a("--finetune-after-trial", type=int, default=0)
    a("--no-multi-process", action="store_false", dest="multi_process")
    a("--random-order-actions", action="store_true")
    a("--support-comm-predict", action="store_true")
    a("--sort-metric", type=str, default="max_stage_time")
    a("--finetune-tp-dp-after-trial", action="store_true")
    a("--init-dim", type=str, default="tp")
    a("--num-partners-in-op-mig", type=int, default=1)
    a("--do-not-continue-when-fail", action="store_false", dest="continue_when_fail")
    a("--adaptive-hyper-parameters", type=int, default=5)
    a("--num-of-saved-configs", type=int, default=1)
    a("--simple-prim-mbs", action="store_true")
    a("--simple-prim-mig", action="store_true")
    a("--only-top-1-target", action="store_true")
    a("--consider-collective-memory", action="store_true")
    a("--no-price-overlap", action="store_false", dest="price_overlap")
    a("--save-to-csv", type=str, default=None)
    a("--shapes", type=str, default="reference", choices=["reference", "b200"],
      help="model dimensions written into the plan JSON: the reference's size tables or the B200 ones")


def args_from_namespace(ns: argparse.Namespace) -> SearchArgs:
    known = SearchArgs.__dataclass_fields__.keys()
    kw = {k: v for k, v in vars(ns).items() if k in known and v is not None}
    return SearchArgs(**kw).finalize()


class Stopwatch:
    """Elapsed wall time since the last (re)start, the only timer behaviour the search logic depends on."""

    def __init__(self):
        self.t0 = time.time()

    def start(self):
        self.t0 = time.time()

    def reset(self):
        pass

    def elapsed(self) -> float:
        return time.time() - self.t0


class SearchContext:
    """Database, cost model, visited sets and counters for one search process."""

    def __init__(self, args: SearchArgs, verbose: bool = True):
        self.args = args
        first_mbs = args.micro_batch_size[0]
        self.unique_ops = read_unique_ops(args.profiled_time_path, args.model_name, args.model_size, first_mbs)
        self.full_op_list = expand_op_list(self.unique_ops, args.model_name, args.num_layers)
        self.tunable = tunable_ops(args.model_name, self.unique_ops)
        self.never_recompute = never_recompute_ops(args.model_name)
        db_model = args.model_name
        self.db = ProfileDB(db_model, args.model_size, args.profiled_time_path, args.micro_batch_size, args.max_tp,
                            self.unique_ops, use_reserved=args.consider_reserved_space, verbose=verbose)
        main_f, opt_f = STATE_MULTIPLIERS["gpt" if args.model_name == "scale-layer" else args.model_name]
        shared_space = args.consider_shared_space
        if getattr(args, "shapes", "reference") == "b200" and args.model_name == "resnet":
            # tables measured with this framework's runtime: the Wide-ResNet trains in bf16 with fp32 master weights
            # like the transformers (the weights column holds bf16 bytes), and its fused BatchNorm + add + ReLU op
            # keeps activations of its own, so the reference's aliasing rule for bn3 / downsample does not apply
            main_f, opt_f = STATE_MULTIPLIERS["gpt"]
            shared_space = False
        self.cost = CostModel(self.db, CostOptions(
            memory_limit=args.memory_limit, num_gpus_per_node=args.num_gpus_per_node, main_params_factor=main_f,
            optimizer_factor=opt_f, resharding=args.resharding, consider_shared_space=shared_space,
            consider_reserved_space=args.consider_reserved_space,
            consider_collective_memory=args.consider_collective_memory, support_comm_predict=args.support_comm_predict,
            memory_pred_type=args.memory_pred_type, flex_recompute=args.flex_recompute,
            peak_mem_in_backward=args.peak_mem_in_backward, price_overlap=args.price_overlap,
            never_recompute=self.never_recompute))
        self.rng = random.Random(2)
        self.trial_clock = Stopwatch()
        self.total_clock = Stopwatch()
        self.explored = 0
        self.plan_visited: Dict[tuple, list] = {}
        self.target_visited: Dict[tuple, list] = {}
        self.partner_visited: Dict[tuple, list] = {}
        self.move_memo: Dict[tuple, object] = {}
        self.hit_resources = [0, 0, 0]
        self.unexplored: list = []
        self.explored_plans: list = []
        self.current_min_time = 0.0

    # budgets ---------------------------------------------------------------------------------
    def trial_time_up(self) -> bool:
        if self.args.explored_budget is not None:
            return self.explored >= self.args.explored_budget
        return self.trial_clock.elapsed() >= self.args.time_budget_per_trial

    def total_time_up(self) -> bool:
        if self.args.explored_budget is not None:
            return self.explored >= self.args.explored_budget
        return self.total_clock.elapsed() >= self.args.time_budget_total

    def debug(self, msg: str) -> None:
        if self.args.print_debug_info:
            print(msg)


def is_visited(table: dict, key, target="") -> bool:
    return key in table and target in table[key]


def mark_visited(table: dict, key, target="") -> None:
    table.setdefault(key, []).append(target)


def num_visited(table: dict, key) -> int:
    return len(table.get(key, ()))
