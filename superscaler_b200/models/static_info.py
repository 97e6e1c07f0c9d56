"""Static description of every op by NAME: which state keys it reads / writes and in which layout.

The runtime needs this for ops that live on OTHER ranks (to know what crosses a pipeline boundary and how
it is sharded there) and for resharding inside a stage: before an op runs, every tensor it reads is
brought to the layout the op requires under its own (tp, dp, algo).

This table is the runtime twin of the search-side sharding specs (`search/opinfo.py`, reference:
search/model_ops_info.py:92-150 and the *_tensors_info / required_input_specs attributes of
runtime/megatron/model/flex_ops.py): `Layout(row, col)` with col "split" corresponds to a spec whose hidden
(or head / channel) dimension is divided by tp, col "rep" to R = tp.
"""
from __future__ import annotations

from typing import Dict, Tuple

from ..parallel.relayout import Layout

ROWS = Layout("split", "rep")          # tokens split over dp, features replicated over tp
COLS = Layout("split", "split")        # features (or heads) split over tp
QKV3 = Layout("split", "split", 3)     # fused [Q | K | V] columns, each third split over tp
KV2 = Layout("split", "split", 2)
VEC = Layout("rep", "rep")             # a parameter vector riding with the activations
VEC_COLS = Layout("rep", "split")      # ... sharded over tp (1-D tensors are split along dim 0 by `row`)


def _strip(name: str) -> str:
    """Drops the enc-/dec- prefix and the -1/-2 suffix of T5 decoder attention ops."""
    for pre in ("enc-", "dec-"):
        if name.startswith(pre):
            name = name[len(pre):]
    return name


def _resnet_kind(name: str):
    if name in ("conv1", "bn1", "relu1", "maxpool", "avgpool", "fc"):
        return name
    if name.startswith("block-"):
        return "block-" + name.split("-")[3]
    return None


def op_io(name: str) -> Tuple[Tuple[str, ...], Tuple[str, ...]]:
    """(reads, writes) of an op."""
    rk = _resnet_kind(name)
    if rk is not None:
        if rk == "block-conv1":
            return ("x",), ("x", "residual")
        if rk == "block-downsample":
            return ("x", "residual"), ("x",)
        if rk == "fc":
            return ("x", "labels"), ("loss",)
        if rk == "conv1":
            return ("images",), ("x",)
        return ("x",), ("x",)
    n = _strip(name)
    if name == "encoder-embedding":
        return ("ids",), ("x",)
    if name == "decoder-embedding":
        return ("dec_ids", "x"), ("x", "enc_out")
    if n in ("1st-layernorm", "2nd-layernorm", "3rd-layernorm"):
        return ("x",), ("x", "residual")
    if n in ("final-layernorm",) or name == "final-layernorm":
        return ("x",), ("x",)
    if n in ("attention-qkv", "attention-qkv-1"):
        return ("x",), ("x",)
    if n == "attention-qkv-2":
        return ("x", "enc_out"), ("x", "kv")
    if n in ("attention-score", "attention-score-1"):
        return ("x",), ("x", "value")
    if n == "attention-score-2":
        return ("x", "kv"), ("x", "value")
    if n.startswith("attention-softmax") or n.startswith("attention-dropout"):
        return ("x",), ("x",)
    if n.startswith("attention-context"):
        return ("x", "value"), ("x",)
    if n.startswith("attention-dense") or n == "MLP-GEMM-2" or n == "MLP-GEMM-1":
        return ("x",), ("x", "bias")
    if n.startswith("post-attention-dropout") or n == "post-MLP-dropout":
        return ("x", "bias", "residual"), ("x",)
    if n == "MLP-gelu":
        return ("x", "bias"), ("x",)
    if name in ("gpt-post-process", "t5-post-process"):
        return ("x", "labels", "loss_mask"), ("loss",)
    if name == "bert-post-process":
        return ("x", "labels", "loss_mask", "nsp"), ("loss",)
    if name == "ict-post-process":
        return ("x", "labels"), ("loss",)
    if name == "vit-embedding":
        return ("images",), ("x",)
    if name == "vit-post-process":
        return ("x", "labels"), ("loss",)
    raise KeyError(f"no static info for op {name}")


def required_layouts(name: str, algo: int) -> Dict[str, Layout]:
    """Layout each read key must have when the op starts (keys fed by the data loader are absent)."""
    rk = _resnet_kind(name)
    if rk is not None:
        if rk == "conv1":
            return {}
        return {"x": ROWS, "residual": ROWS} if rk == "block-downsample" else {"x": ROWS}
    n = _strip(name)
    if name in ("encoder-embedding", "vit-embedding"):
        return {}
    if name == "decoder-embedding":
        return {"x": ROWS}
    if "layernorm" in n:
        return {"x": ROWS}
    if n in ("attention-qkv", "attention-qkv-1"):
        return {"x": ROWS if algo == 0 else COLS}
    if n == "attention-qkv-2":
        return {"x": ROWS, "enc_out": ROWS}
    if n in ("attention-score", "attention-score-1"):
        return {"x": QKV3}
    if n == "attention-score-2":
        return {"x": COLS, "kv": KV2}
    if n.startswith("attention-softmax") or n.startswith("attention-dropout"):
        return {"x": COLS}
    if n.startswith("attention-context"):
        return {"x": COLS, "value": COLS}
    if n.startswith("attention-dense") or n == "MLP-GEMM-2":
        return {"x": COLS if algo == 0 else ROWS}
    if n == "MLP-GEMM-1":
        return {"x": ROWS if algo == 0 else COLS}
    if n.startswith("post-attention-dropout") or n == "post-MLP-dropout":
        return {"x": ROWS, "bias": VEC, "residual": ROWS}
    if n == "MLP-gelu":
        return {"x": COLS, "bias": VEC_COLS}
    if name in ("gpt-post-process", "t5-post-process", "bert-post-process", "vit-post-process", "ict-post-process"):
        return {"x": ROWS}
    raise KeyError(f"no static info for op {name}")


def produced_layouts(name: str, algo: int) -> Dict[str, Layout]:
    rk = _resnet_kind(name)
    if rk is not None:
        if rk == "fc":
            return {}
        return {"x": ROWS, "residual": ROWS} if rk == "block-conv1" else {"x": ROWS}
    n = _strip(name)
    if name in ("encoder-embedding", "vit-embedding"):
        return {"x": ROWS}
    if name == "decoder-embedding":
        return {"x": ROWS, "enc_out": ROWS}
    if n in ("1st-layernorm", "2nd-layernorm", "3rd-layernorm"):
        return {"x": ROWS, "residual": ROWS}
    if "final-layernorm" in n:
        return {"x": ROWS}
    if n in ("attention-qkv", "attention-qkv-1"):
        return {"x": QKV3 if algo == 0 else Layout("split", "rep", 3)}
    if n == "attention-qkv-2":
        return {"x": COLS, "kv": KV2}
    if n.startswith("attention-score"):
        return {"x": COLS, "value": COLS}
    if n.startswith("attention-softmax") or n.startswith("attention-dropout") or n.startswith("attention-context"):
        return {"x": COLS}
    if n.startswith("attention-dense") or n == "MLP-GEMM-2":
        return {"x": ROWS, "bias": VEC} if algo == 0 else {"x": COLS, "bias": VEC_COLS}
    if n == "MLP-GEMM-1":
        return {"x": COLS, "bias": VEC_COLS} if algo == 0 else {"x": ROWS, "bias": VEC}
    if n.startswith("post-attention-dropout") or n == "post-MLP-dropout":
        return {"x": ROWS}
    if n == "MLP-gelu":
        return {"x": COLS}
    if name in ("gpt-post-process", "t5-post-process", "bert-post-process", "vit-post-process", "ict-post-process"):
        return {}
    raise KeyError(f"no static info for op {name}")


DATA_KEYS = ("ids", "dec_ids", "labels", "loss_mask", "images", "enc_lens", "types", "nsp")


def live_keys_before(op_names, cut: int):
    """State keys that must cross a boundary placed before op `cut` (data-loader keys never travel)."""
    written = set()
    for n in op_names[:cut]:
        written.update(op_io(n)[1])
    live, killed = [], set()
    for n in op_names[cut:]:
        r, w = op_io(n)
        for k in r:
            if k not in killed and k in written and k not in live and k not in DATA_KEYS:
                live.append(k)
        killed.update(w)
    return live
