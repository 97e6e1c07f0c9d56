"""Plan data model, model-size tables, plan JSON I/O and initial-plan generators (CPU only).

The plan JSON is the contract between the search and the runtime and keeps the reference's schema
(written by search/aceso_utils.py:137-211, read by runtime/megatron/arguments.py:90-124):
``model_name, model_size, num_layers, <model shape keys>, global_batch_size, micro_batch_size, num_stages,
num_gpus[stage], checkpoint_activations[stage], resharding_stages[stage], num_ops_in_each_stage[stage],
model_parallel_size_of_each_op[stage][op], data_parallel_size_of_each_op[stage][op],
recompute_ops[stage][op], algo_of_each_op[stage][op]``.
``micro_batch_size`` is the stage-aggregate micro-batch: an op with dp = d sees micro_batch_size / d samples.
"""
from __future__ import annotations

import csv
import json
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

BIG = 2 ** 30
SMALL = -2 ** 30

# model_size -> (blocks per group, base channels, width factor, parameter dtype)
RESNET_SIZES: Dict[str, tuple] = {
    "250M": ([3, 4, 6, 3], 160, 2, "fp32"),
    "500M": ([3, 4, 6, 3], 224, 2, "fp32"),
    "1B": ([3, 4, 6, 3], 320, 2, "fp32"),
    "2B": ([3, 4, 6, 3], 448, 2, "fp32"),
    "4B": ([3, 4, 6, 3], 640, 2, "fp32"),
    "6_8B": ([3, 4, 6, 3], 320, 16, "fp32"),
    "13B": ([3, 4, 23, 3], 320, 16, "fp32"),
}
# model_size -> (layers, seq, hidden, ffn, heads, kv_channels, vocab, dtype)
GPT_SIZES: Dict[str, tuple] = {
    "350M": (24, 2048, 1024, 4096, 16, 64, 51200, "fp16"),
    "1_3B": (24, 2048, 2048, 8192, 32, 64, 51200, "fp16"),
    "2_6B": (32, 2048, 2560, 10240, 32, 80, 51200, "fp16"),
    "6_7B": (32, 2048, 4096, 16384, 32, 128, 51200, "fp16"),
    "13B": (40, 2048, 5120, 20480, 40, 128, 51200, "fp16"),
    "scale-layer": (1, 2048, 512, 2048, 8, 64, 51200, "fp16"),
}
# model_size -> (layers, enc seq, dec seq, hidden, ffn, heads, kv_channels, vocab, dtype)
T5_SIZES: Dict[str, tuple] = {
    "770M": (24, 2048, 512, 1024, 4096, 16, 64, 30592, "fp16"),
    "3B": (24, 2048, 512, 1024, 16384, 32, 128, 30592, "fp16"),
    "6B": (24, 2048, 512, 1024, 32768, 64, 128, 30592, "fp16"),
    "11B": (24, 2048, 512, 1024, 65536, 128, 128, 30592, "fp16"),
    "22B": (48, 2048, 512, 1024, 65536, 128, 128, 30592, "fp16"),
}
# Shapes profiled on B200 under the same database file names (the benchmark's model definitions differ from the
# reference tables above: GPT-3 1.3B uses 16 heads of 128; T5 770M uses encoder 512 / decoder 128 tokens, vocab 32128)
B200_GPT_SIZES: Dict[str, tuple] = {
    "1_3B": (24, 2048, 2048, 8192, 16, 128, 51200, "bf16"),
    # the attention kernels take heads of 64 or 128: 2.6B runs 20 heads of 128 instead of 32 of 80
    "2_6B": (32, 2048, 2560, 10240, 20, 128, 51200, "bf16"),
}
B200_T5_SIZES: Dict[str, tuple] = {
    "770M": (24, 512, 128, 1024, 4096, 16, 64, 32128, "bf16"),
}
# Encoder-only families that exist only in this framework (the reference has no op-list BERT / ViT):
# model_size -> (layers, seq, hidden, ffn, heads, kv_channels, vocab, dtype)
BERT_SIZES: Dict[str, tuple] = {
    "110M": (12, 512, 768, 3072, 12, 64, 30592, "bf16"),
    "340M": (24, 512, 1024, 4096, 16, 64, 30592, "bf16"),
    "1_3B": (24, 512, 2048, 8192, 16, 128, 30592, "bf16"),
}
# model_size -> (layers, image size, patch, hidden, ffn, heads, kv_channels, classes, dtype)
VIT_SIZES: Dict[str, tuple] = {
    "base": (12, 224, 16, 768, 3072, 12, 64, 1000, "bf16"),
    "large": (24, 224, 16, 1024, 4096, 16, 64, 1000, "bf16"),
    "huge": (32, 224, 16, 1280, 5120, 20, 64, 1000, "bf16"),    # 16 x 16 patches (the published huge model uses 14 x 14)
}
# multiples of the weight bytes held besides weights and gradients: (fp32 main params, optimizer state)
STATE_MULTIPLIERS = {"resnet": (0, 2), "gpt": (2, 4), "t5": (2, 4), "bert": (2, 4), "vit": (2, 4)}


@dataclass
class StagePlan:
    """One pipeline stage: a contiguous slice of the op list with per-op parallel degrees."""
    index: int
    num_stages_behind: int
    num_gpus: int
    ops: List[str]
    recompute_ops: List[int]
    tp_size: List[int]
    dp_size: List[int]
    algo: List[int]

    def clone(self) -> "StagePlan":
        return StagePlan(self.index, self.num_stages_behind, self.num_gpus, list(self.ops),
                         list(self.recompute_ops), list(self.tp_size), list(self.dp_size), list(self.algo))


@dataclass
class Plan:
    """A full parallel plan plus the cost-model annotations the search attaches to it."""
    global_bs: int
    micro_bs: int
    stages: List[StagePlan]
    num_stages: int
    history: str = ""
    time_list: List[float] = field(default_factory=list)
    memory_list: List[float] = field(default_factory=list)
    compute_time_list: List[float] = field(default_factory=list)
    total_gpu_time: float = 0
    ideal_time_per_gpu: List[float] = field(default_factory=list)
    eff_loss_time_per_gpu: List[float] = field(default_factory=list)
    recomp_time_per_gpu: List[float] = field(default_factory=list)
    efficient_time_list: List[float] = field(default_factory=list)
    adaptive_times: int = 0

    def clone(self) -> "Plan":
        return Plan(self.global_bs, self.micro_bs, [s.clone() for s in self.stages], self.num_stages, self.history,
                    list(self.time_list), list(self.memory_list), list(self.compute_time_list), self.total_gpu_time,
                    list(self.ideal_time_per_gpu), list(self.eff_loss_time_per_gpu), list(self.recomp_time_per_gpu),
                    list(self.efficient_time_list), self.adaptive_times)

    # identity of the parallelisation decisions (what the visited-sets key on)
    def key(self) -> tuple:
        return (tuple(len(s.ops) for s in self.stages), tuple(tuple(s.tp_size) for s in self.stages),
                tuple(tuple(s.dp_size) for s in self.stages), tuple(tuple(s.recompute_ops) for s in self.stages),
                self.micro_bs, tuple(tuple(s.algo) for s in self.stages))


def build_plan(num_ops_list: Sequence[int], tp_flat: Sequence[int], dp_flat: Sequence[int],
               recompute_flat: Sequence[int], micro_bs: int, global_bs: int, full_op_list: Sequence[str],
               algo_flat: Sequence[int]) -> Plan:
    """Cuts flat per-op lists into stages; a stage's GPU count is tp * dp of its first op."""
    stages = []
    start = 0
    n = len(num_ops_list)
    for i, cnt in enumerate(num_ops_list):
        end = start + cnt
        stages.append(StagePlan(index=i, num_stages_behind=n - 1 - i, num_gpus=tp_flat[start] * dp_flat[start],
                                ops=list(full_op_list[start:end]), recompute_ops=list(recompute_flat[start:end]),
                                tp_size=list(tp_flat[start:end]), dp_size=list(dp_flat[start:end]),
                                algo=list(algo_flat[start:end])))
        start = end
    return Plan(global_bs=global_bs, micro_bs=micro_bs, stages=stages, num_stages=n)


def plan_to_dict(plan: Plan, model_name: str, model_size: str, num_layers: int, shapes: str = "reference") -> dict:
    """Plan JSON.  shapes = "reference": the model dimensions of the reference's size tables (byte-compatible with
    its plan files); "b200": the B200_* tables (e.g. GPT-3 1.3B with 16 heads of 128) with every dimension the
    runtime needs spelled out."""
    if model_name == "scale-layer":
        model_name, model_size = "gpt", "scale-layer"
    d: dict = {"model_name": model_name, "model_size": model_size}
    if model_name == "resnet":
        layers, in_channels, width_factor, _ = RESNET_SIZES[model_size]
        d["num_layers"] = layers
        d["in_channels"] = in_channels
        d["width_factor"] = width_factor
    elif model_name == "gpt":
        _, seq, hidden, _ffn, heads, _kv, _vocab, _ = GPT_SIZES[model_size]
        d["num_layers"] = num_layers
        d["seq_length"] = seq
        d["max_position_embeddings"] = seq
        d["num_attention_heads"] = heads
        d["hidden_size"] = hidden
        if shapes == "b200" and model_size in B200_GPT_SIZES:
            _, seq, hidden, ffn, heads, kv, vocab, _ = B200_GPT_SIZES[model_size]
            d.update(num_attention_heads=heads, kv_channels=kv, ffn_hidden_size=ffn, vocab_size=vocab)
    elif model_name == "t5":
        _, enc_seq, dec_seq, hidden, ffn, heads, kv, _vocab, _ = T5_SIZES[model_size]
        if shapes == "b200" and model_size in B200_T5_SIZES:
            _, enc_seq, dec_seq, hidden, ffn, heads, kv, _vocab, _ = B200_T5_SIZES[model_size]
        d["num_layers"] = num_layers
        d["encoder_seq_length"] = enc_seq
        d["decoder_seq_length"] = dec_seq
        d["max_position_embeddings"] = enc_seq
        d["num_attention_heads"] = heads
        d["kv_channels"] = kv
        d["hidden_size"] = hidden
        d["ffn_hidden_size"] = ffn
        if shapes == "b200":
            d["vocab_size"] = _vocab
            # the benchmark's T5: ReLU feed-forward, relative-position buckets instead of nothing but absolute positions
            d["activation"] = "relu"
            d["relative_position_bias"] = True
            d["relative_attention_num_buckets"] = 32
    elif model_name == "bert":
        _, seq, hidden, ffn, heads, kv, vocab, _ = BERT_SIZES[model_size]
        d.update(num_layers=num_layers, seq_length=seq, max_position_embeddings=seq, num_attention_heads=heads,
                 hidden_size=hidden, kv_channels=kv, ffn_hidden_size=ffn, vocab_size=vocab)
    elif model_name == "vit":
        _, image, patch, hidden, ffn, heads, kv, classes, _ = VIT_SIZES[model_size]
        d.update(num_layers=num_layers, image_size=image, patch_dim=patch, num_classes=classes,
                 seq_length=(image // patch) ** 2 + 1, max_position_embeddings=(image // patch) ** 2 + 1,
                 num_attention_heads=heads, hidden_size=hidden, kv_channels=kv, ffn_hidden_size=ffn)
    else:
        raise ValueError(f"unsupported model {model_name}")
    d["global_batch_size"] = plan.global_bs
    d["micro_batch_size"] = plan.micro_bs
    d["num_stages"] = plan.num_stages
    d["num_gpus"] = [s.num_gpus for s in plan.stages]
    d["checkpoint_activations"] = [max(s.recompute_ops) > 0 for s in plan.stages]
    d["resharding_stages"] = [
        (max(s.tp_size) != min(s.tp_size)) or (max(s.dp_size) != min(s.dp_size)) or (max(s.algo) != min(s.algo))
        for s in plan.stages]
    d["num_ops_in_each_stage"] = [len(s.ops) for s in plan.stages]
    d["model_parallel_size_of_each_op"] = [s.tp_size for s in plan.stages]
    d["data_parallel_size_of_each_op"] = [s.dp_size for s in plan.stages]
    d["recompute_ops"] = [s.recompute_ops for s in plan.stages]
    d["algo_of_each_op"] = [s.algo for s in plan.stages]
    return d


def save_plan(plan: Plan, path: str, model_name: str, model_size: str, num_layers: int,
              shapes: str = "reference") -> None:
    with open(path, "w") as f:
        json.dump(plan_to_dict(plan, model_name, model_size, num_layers, shapes), f, indent=4)


def plan_from_dict(d: dict, full_op_list: Sequence[str]) -> Plan:
    flat = lambda key: [x for stage in d[key] for x in stage]  # noqa: E731
    return build_plan(d["num_ops_in_each_stage"], flat("model_parallel_size_of_each_op"),
                      flat("data_parallel_size_of_each_op"), flat("recompute_ops"), d["micro_batch_size"],
                      d["global_batch_size"], full_op_list, flat("algo_of_each_op"))


def load_plan(path: str, full_op_list: Sequence[str]) -> Tuple[Plan, dict]:
    with open(path) as f:
        d = json.load(f)
    return plan_from_dict(d, full_op_list), d


def write_stage_info_csv(plan: Plan, reserved: Sequence[float], path: str) -> None:
    rows = [["stage-index", "time", "memory(total)", "memory(normal)", "memory(reserved)"]]
    for i in range(plan.num_stages):
        rows.append([f"stage-{i}", f"{plan.time_list[i]:.2f}", f"{plan.memory_list[i]:.2f}",
                     f"{(plan.memory_list[i] - reserved[i]):.2f}", f"{reserved[i]:.2f}"])
    with open(path, "w", newline="") as f:
        csv.writer(f).writerows(rows)


# ------------------------------------------------------------------------------------------------
# legality and initial plans
# ------------------------------------------------------------------------------------------------
def is_legal(plan: Plan, num_gpus: int, gpus_per_node: int, num_nodes: int) -> bool:
    """Stage sizes in {1,2,4,8}, all GPUs used, and every node boundary coincides with a stage boundary."""
    running = []
    total = 0
    for s in plan.stages:
        if s.num_gpus not in (1, 2, 4, 8):
            return False
        total += s.num_gpus
        running.append(total)
    if total != num_gpus:
        return False
    return all(gpus_per_node * k in running for k in range(1, num_nodes + 1))


def _double_round_robin(num_stages: int, num_gpus: int, max_tp: int) -> Optional[List[int]]:
    gpus = [1] * num_stages
    progressed = True
    while sum(gpus) < num_gpus and progressed:
        progressed = False
        for i in range(num_stages):
            if sum(gpus) < num_gpus and gpus[i] < max_tp and gpus[i] <= (num_gpus - sum(gpus)):
                gpus[i] *= 2
                progressed = True
    return gpus if sum(gpus) == num_gpus else None


def _even_ops(num_ops: int, num_stages: int) -> List[int]:
    per = [num_ops // num_stages] * num_stages
    per[-1] += num_ops - num_stages * (num_ops // num_stages)
    return per


def balanced_plan(full_op_list, num_stages, *, num_gpus, global_bs, micro_bs, max_tp, flex_recompute=True,
                  init_dim="tp") -> Optional[Plan]:
    """Even op split; GPUs doubled round-robin over the stages; the whole stage starts as pure TP (or tp2 x dp)."""
    gpus = _double_round_robin(num_stages, num_gpus, max_tp)
    if gpus is None:
        return None
    n = len(full_op_list)
    per = _even_ops(n, num_stages)
    tp, dp = [], []
    for i in range(num_stages):
        if init_dim == "tp":
            tp += [gpus[i]] * per[i]
            dp += [1] * per[i]
        elif init_dim == "dp":
            dp += [gpus[i] // 2] * per[i]
            tp += [2] * per[i]
    rc = [0] * n if flex_recompute else [1] * n
    return build_plan(per, tp, dp, rc, micro_bs, global_bs, full_op_list, [0] * n)


def imbalanced_gpu_plan(full_op_list, num_stages, *, num_gpus, global_bs, micro_batch_sizes, max_tp) -> Plan:
    """Even op split; later stages are given GPUs first, raising the micro-batch when dp would not divide it."""
    n = len(full_op_list)
    per = _even_ops(n, num_stages)
    gpus = [1] * num_stages
    left = num_gpus - num_stages
    micro_bs = micro_batch_sizes[0]
    mbs_i = 0
    while left > 0:
        found = False
        for k in range(num_stages):
            s = num_stages - 1 - k
            over = gpus[s] * 2 // max_tp
            if gpus[s] <= left and (over == 0 or micro_bs // over in micro_batch_sizes):
                left -= gpus[s]
                gpus[s] *= 2
                found = True
                break
        if not found:
            mbs_i += 1
            assert mbs_i < len(micro_batch_sizes)
            micro_bs = micro_batch_sizes[mbs_i]
    tp, dp = [], []
    for i in range(num_stages):
        if gpus[i] <= max_tp:
            tp += [gpus[i]] * per[i]
            dp += [1] * per[i]
        else:
            tp += [max_tp] * per[i]
            dp += [gpus[i] // max_tp] * per[i]
    return build_plan(per, tp, dp, [0] * n, micro_bs, global_bs, full_op_list, [0] * n)


def imbalanced_op_plan(full_op_list, num_stages, *, model_name, num_layers, num_gpus, global_bs, micro_bs, max_tp,
                       flex_recompute=True) -> Optional[Plan]:
    """One layer per stage except one stage that takes all the rest (first for ResNet, last for GPT)."""
    gpus = _double_round_robin(num_stages, num_gpus, max_tp)
    if gpus is None:
        return None
    n = len(full_op_list)
    layers = [1] * num_stages
    if model_name == "resnet":
        layers[0] += 33 - sum(layers)
        per = [l * 8 for l in layers]
        per[0] += 4
        per[-1] += 2
    else:
        layers[-1] += num_layers - sum(layers)
        per = [l * 13 for l in layers]
        per[0] += 1
        per[-1] += 2
    tp, dp = [], []
    for i in range(num_stages):
        tp += [gpus[i]] * per[i]
        dp += [1] * per[i]
    rc = [1] * n if flex_recompute else [0] * n
    return build_plan(per, tp, dp, rc, micro_bs, global_bs, full_op_list, [0] * n)


def single_gpu_plan(full_op_list, *, global_bs, micro_bs, recompute=True, never_recompute=()) -> Plan:
    """The fixed 1-GPU plan used for the 1-GPU points (reference: search/single_gpu_configs/*.json)."""
    n = len(full_op_list)
    rc = [0 if (not recompute or op in never_recompute) else 1 for op in full_op_list]
    return build_plan([n], [1] * n, [1] * n, rc, micro_bs, global_bs, full_op_list, [0] * n)
