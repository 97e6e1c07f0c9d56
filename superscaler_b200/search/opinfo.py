"""Op metadata for the CPU side: op lists, TP-tunable ops, never-recompute ops, sharding specs and the
resharding decision between a producer spec and a consumer spec.

A spec is ``{"R": replicas, "V": partial-value copies, "dims": [parts of dim 0, dim 1, dim 2]}`` of the
logical activation (``[s, b, h]`` for transformers, ``[b, c, h*w]`` for ResNet), as in the reference
(search/model_ops_info.py:92-150).  It must agree with what the runtime ops really produce and consume.
"""
from __future__ import annotations

import csv
from typing import List, Optional, Sequence, Tuple

GPT_TUNABLE = ["encoder-embedding", "enc-attention-qkv", "enc-attention-dense", "enc-MLP-GEMM-1", "enc-MLP-GEMM-2"]
T5_TUNABLE = GPT_TUNABLE + ["dec-attention-qkv-1", "dec-attention-dense-1", "dec-attention-qkv-2",
                            "dec-attention-dense-2", "dec-MLP-GEMM-1", "dec-MLP-GEMM-2"]
NEVER_RECOMPUTE = {
    "gpt": ["encoder-embedding", "gpt-post-process"],
    "scale-layer": ["encoder-embedding", "gpt-post-process"],
    "t5": ["encoder-embedding", "decoder-embedding", "t5-post-process"],
    "resnet": ["conv1"],
    "bert": ["encoder-embedding", "bert-post-process"],
    "vit": ["vit-embedding", "vit-post-process"],
}
# families laid out like GPT: one head op, 13 ops per layer, final LayerNorm + post-process
GPT_LIKE = ("gpt", "scale-layer", "bert", "vit")


def read_unique_ops(profile_dir: str, model_name: str, model_size: str, first_mbs: int) -> List[str]:
    """Op names in database order, from the tp1 / algo0 table of the smallest micro-batch."""
    if model_name == "scale-layer":
        path = f"{profile_dir}gpt_scale-layer_mbs{first_mbs}_tp1_algo0.csv"
    else:
        size = "11B" if (model_name == "t5" and model_size == "22B") else model_size
        path = f"{profile_dir}{model_name}_{size}_mbs{first_mbs}_tp1_algo0.csv"
    with open(path) as f:
        rows = list(csv.reader(f))
    return [r[0] for r in rows[1:]]


def expand_op_list(unique_ops: Sequence[str], model_name: str, num_layers: int) -> List[str]:
    """Full op list: head + layer ops x layers + tail (GPT), encoder / decoder blocks (T5), as-is (ResNet)."""
    u = list(unique_ops)
    if model_name in GPT_LIKE:
        return u[:1] + u[1:14] * num_layers + u[14:]
    if model_name == "t5":
        return u[:1] + u[1:14] * num_layers + u[14:15] + u[15:16] + u[16:37] * num_layers + u[37:]
    if model_name == "resnet":
        return u
    raise ValueError(f"unsupported model {model_name}")


def tunable_ops(model_name: str, unique_ops: Sequence[str]) -> List[str]:
    if model_name in ("gpt", "scale-layer", "bert"):
        return list(GPT_TUNABLE)
    if model_name == "vit":
        return [op for op in GPT_TUNABLE if op != "encoder-embedding"]     # the patch projection is never sharded
    if model_name == "t5":
        return list(T5_TUNABLE)
    if model_name == "resnet":
        return [op for op in unique_ops if "conv" in op or "downsample" in op]
    raise ValueError(f"unsupported model {model_name}")


def never_recompute_ops(model_name: str) -> List[str]:
    return list(NEVER_RECOMPUTE[model_name])


def _spec(r, v, dims):
    return {"R": r, "V": v, "dims": dims}


def op_spec(op: str, tp: int, dp: int, algo: int, as_input: bool) -> Optional[dict]:
    """Required input spec (as_input) or produced output spec of an op under (tp, dp, algo)."""
    replicated_b = _spec(tp, 1, [1, dp, 1])       # replicated over tp, batch split over dp
    split_h = _spec(1, 1, [1, dp, tp])            # hidden dim split over tp
    heads = _spec(1, 1, [dp, tp, 1])              # [b, np, ...] attention layout
    if op in ("encoder-embedding", "vit-embedding"):
        return None if as_input else replicated_b
    if op in ("enc-1st-layernorm", "enc-2nd-layernorm", "enc-post-attention-dropout", "enc-post-MLP-dropout"):
        return replicated_b
    if op == "final-layernorm":
        return replicated_b if as_input else _spec(tp, 1, [dp, 1, 1])
    if op in ("enc-attention-qkv", "enc-MLP-GEMM-1"):
        column = algo == 0
        if column:
            return replicated_b if as_input else split_h
        return split_h if as_input else replicated_b
    if op == "enc-attention-score":
        return split_h if as_input else heads
    if op in ("enc-attention-softmax", "enc-attention-dropout"):
        return heads
    if op == "enc-attention-context":
        return heads if as_input else split_h
    if op in ("enc-attention-dense", "enc-MLP-GEMM-2"):
        row = algo == 0
        if row:
            return split_h if as_input else replicated_b
        return replicated_b if as_input else split_h
    if op == "enc-MLP-gelu":
        return split_h
    if op in ("gpt-post-process", "bert-post-process", "vit-post-process"):
        return _spec(tp, 1, [dp, 1, 1]) if as_input else None
    if any(k in op for k in ("conv", "downsample", "bn", "relu", "pool", "fc")):
        return _spec(tp, 1, [dp, 1, 1])
    return None


def same_spec(a: Optional[dict], b: Optional[dict]) -> bool:
    if a is None or b is None:
        return True
    return a["R"] == b["R"] and a["V"] == b["V"] and all(x == y for x, y in zip(a["dims"], b["dims"]))


def reshard_primitives(src: Optional[dict], dst: Optional[dict]) -> Tuple[Optional[str], Optional[str], int]:
    """(forward collective, backward collective, group size) that turns layout `src` into `dst`.

    replicas -> split dim : split / all-gather          partial -> replicas : all-reduce / -
    partial  -> split dim : reduce-scatter / all-gather  split -> replicas   : all-gather / split
    split dim i -> dim j  : all-to-all / all-to-all
    (reference: search/aceso_cost_model.py:200-245, runtime/megatron/mpu/mappings.py:382-468)."""
    if same_spec(src, dst):
        return None, None, 0
    sd, dd = src["dims"], dst["dims"]
    if src["R"] > dst["R"]:
        for i in range(len(sd)):
            if sd[i] < dd[i]:
                assert src["R"] % dst["R"] == 0
                return "split", "all_gather", src["R"] // dst["R"]
    elif src["V"] > dst["V"]:
        if src["R"] < dst["R"]:
            assert src["V"] % dst["V"] == 0
            return "all_reduce", None, src["V"] // dst["V"]
        for i in range(len(sd)):
            if sd[i] < dd[i]:
                assert src["V"] % dst["V"] == 0
                return "reduce_scatter", "all_gather", src["V"] // dst["V"]
    else:
        for i in range(len(sd)):
            if sd[i] > dd[i]:
                if src["R"] < dst["R"]:
                    assert sd[i] % dd[i] == 0
                    return "all_gather", "split", sd[i] // dd[i]
                for j in range(len(sd)):
                    if j != i and sd[j] < dd[j]:
                        assert sd[i] % dd[i] == 0
                        return "all_to_all", "all_to_all", sd[i] // dd[i]
    return None  # unreachable for legal plans; mirrors the reference, which returns nothing here
