"""Wide-ResNet (bottleneck) as a flat op list with the reference's op names
(runtime/megatron/model/flex_resnet.py:19-74): `conv1 bn1 relu1 maxpool`, then for every block of the groups
[3, 4, 6, 3] the 8 ops `block-g-b-{conv1, bn1, conv2, bn2, conv3, bn3, downsample, relu}`, then `avgpool fc`
(134 ops).  Group g uses base channels C = in_channels * 2^g: conv1 1x1 -> C, conv2 3x3 (stride 2 in the first
block of groups 1..3) -> C * width_factor, conv3 1x1 -> 4C; `downsample` adds the residual (through a strided
1x1 convolution + BatchNorm in the first block of a group).

Activations are NHWC bf16.  Tensor parallelism of a convolution: algo 0 splits the output channels and
all-gathers them, algo 1 splits the input channels and all-reduces (flex_ops.py:1461-1550); activations between
ops are replicated over the TP group.  BatchNorm statistics are local to a data-parallel rank, as in the reference.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Sequence

import torch

from ..ops import conv as C
from ..ops import functional as F
from ..parallel import mappings as M
from .base import Env, Op, OpInfo
from .fused import FusedGroup


@dataclass
class ResNetConfig:
    blocks: Sequence[int] = (3, 4, 6, 3)
    in_channels: int = 320
    width_factor: int = 2
    num_classes: int = 1000
    image_size: int = 224
    inner_relu: bool = True      # ReLU after bn1 / bn2 of a block (standard bottleneck; the reference has none)
    bn_eps: float = 1e-5
    bn_momentum: float = 0.1
    init_std: float = 0.02
    hidden_dropout: float = 0.0
    attention_dropout: float = 0.0


def resnet_op_names(cfg: ResNetConfig) -> List[str]:
    names = ["conv1", "bn1", "relu1", "maxpool"]
    for g, nb in enumerate(cfg.blocks):
        for b in range(nb):
            names += [f"block-{g}-{b}-{k}" for k in ("conv1", "bn1", "conv2", "bn2", "conv3", "bn3", "downsample", "relu")]
    return names + ["avgpool", "fc"]


def resnet_layer_of(index: int, cfg: ResNetConfig) -> int:
    return -1 if index < 4 else (index - 4) // 8


def _block_geometry(cfg: ResNetConfig, g: int, b: int):
    """(input channels, base channels, stride, input width) of block (g, b)."""
    base = cfg.in_channels * 2 ** g
    width = cfg.image_size // 4 // (2 ** g)
    stride = 2 if (g > 0 and b == 0) else 1
    if b == 0:
        cin = cfg.in_channels if g == 0 else cfg.in_channels * 2 ** (g - 1) * 4
        win = width * stride
    else:
        cin, win = base * 4, width
    return cin, base, stride, win


class ConvOp(Op):
    reads = ("x",)
    writes = ("x",)

    def __init__(self, info, env, cin, cout, k, stride, pad, keep_residual=False, key="conv"):
        super().__init__(info, env)
        self.cin, self.cout, self.k, self.stride, self.pad, self.key = cin, cout, k, stride, pad, key
        self.keep_residual = keep_residual
        if keep_residual:
            self.writes = ("x", "residual")

    def declare(self):
        tp, kk = self.pl.tp, self.k * self.k
        if self.info.algo == 0 or tp == 1:
            kpad = C._pad8(kk * self.cin)
            self.param_spec(f"{self.key}.weight", (self.cout // tp, kpad), "kaiming", full_shape=(self.cout, kpad),
                            shard_dim=0)
        else:
            self.param_spec(f"{self.key}.weight", (self.cout, kk, self.cin // tp), "kaiming",
                            full_shape=(self.cout, kk, self.cin), shard_dim=2)

    def conv(self, x):
        w = self.p(f"{self.key}.weight")
        if self.info.algo == 0 or self.pl.tp == 1:
            y = C.conv2d(M.copy_to_group(x, self.tp_group), w, self.k, self.k, self.stride, self.pad)
            return M.gather_from_group(y, 3, self.tp_group)
        xs = M.split_to_group(x, 3, self.tp_group)
        y = C.conv2d(xs, w.view(w.shape[0], -1), self.k, self.k, self.stride, self.pad)
        return M.reduce_from_group(y, self.tp_group)

    def forward(self, st):
        x = st["x"] if "x" in st else st.pop("images")   # the stem reads the data loader's images
        if self.keep_residual:
            st["residual"] = x
        st["x"] = self.conv(x)


class BNOp(Op):
    def __init__(self, info, env, channels, relu=False, key="bn"):
        super().__init__(info, env)
        self.ch, self.relu, self.key = channels, relu, key
        self.run_mean = self.run_var = None

    def declare(self):
        self.param_spec(f"{self.key}.weight", (self.ch,), "ones", weight_decay=False, fp32=True)
        self.param_spec(f"{self.key}.bias", (self.ch,), "zeros", weight_decay=False, fp32=True)

    def _buffers(self, dev):
        if self.run_mean is None:
            self.run_mean = torch.zeros(self.ch, dtype=torch.float32, device=dev)
            self.run_var = torch.ones(self.ch, dtype=torch.float32, device=dev)
        return self.run_mean, self.run_var

    def apply(self, x, residual=None, relu=None):
        c = self.env.cfg
        rm, rv = self._buffers(x.device)
        if not self.env.training:
            # evaluation: running statistics, buffers untouched (torch.nn.BatchNorm2d.eval() in the reference)
            return C.batch_norm_inference(x, self.p(f"{self.key}.weight"), self.p(f"{self.key}.bias"), rm, rv,
                                          residual, c.bn_eps, self.relu if relu is None else relu)
        return C.batch_norm(x, self.p(f"{self.key}.weight"), self.p(f"{self.key}.bias"), residual, rm, rv, c.bn_eps,
                            c.bn_momentum, self.relu if relu is None else relu)

    def forward(self, st):
        st["x"] = self.apply(st["x"])


class ReLUOp(Op):
    def forward(self, st):
        x = st["x"]
        st["x"] = F.bias_act(x.reshape(-1, x.shape[-1]), None, F.ACT_RELU).view(x.shape)


class MaxPoolOp(Op):
    def forward(self, st):
        st["x"] = C.max_pool_3x3_s2(st["x"])


class DownsampleOp(Op):
    """x + residual, where the residual first passes a strided 1x1 convolution + BatchNorm in the first block of a
    group (reference: the recv_residual branch of ParallelConvOp.forward)."""
    reads = ("x", "residual")
    writes = ("x",)

    def __init__(self, info, env, cin, cout, stride, project):
        super().__init__(info, env)
        self.project = project
        if project:
            self.conv_op = ConvOp(info, env, cin, cout, 1, stride, 0, key="downsample.conv")
            self.bn_op = BNOp(info, env, cout, key="downsample.bn")

    def declare(self):
        if self.project:
            self.conv_op.declare()
            self.bn_op.declare()
            self._names.update(self.conv_op._names)
            self._names.update(self.bn_op._names)

    def shortcut(self, st):
        r = st.pop("residual")
        if self.project:
            r = self.bn_op.apply(self.conv_op.conv(r))
        return r

    def forward(self, st):
        x = st["x"]
        r = self.shortcut(st)
        st["x"] = F_add(x, r)


def F_add(a, b):
    if a.is_cuda:
        from ..ops import native
        return _AddFn.apply(a, b)
    return a + b


class _AddFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, b):
        from ..ops import native
        return native.ext().elementwise(F.EW_ADD, a.contiguous(), b.contiguous(), None, 0.0, 0)

    @staticmethod
    def backward(ctx, g):
        return g, g


class AvgPoolOp(Op):
    def forward(self, st):
        st["x"] = C.global_avg_pool(st["x"])


class FCLossOp(Op):
    """Classifier + mean cross entropy of the micro-batch (the reference computes the loss outside the op list,
    runtime/pretrain_resnet.py:62-70)."""
    reads = ("x", "labels")
    writes = ("loss", "logits")

    def __init__(self, info, env, cin, classes):
        super().__init__(info, env)
        self.cin, self.classes = cin, classes

    def declare(self):
        self.param_spec("fc.weight", (self.classes, self.cin), "normal", std=self.env.cfg.init_std)
        self.param_spec("fc.bias", (self.classes,), "zeros", weight_decay=False)

    def forward(self, st):
        logits = F.linear(st["x"], self.p("fc.weight"), self.p("fc.bias"))
        if "labels" not in st:            # inference: the class scores (Trainer.embed returns them)
            st["logits"] = logits
            return
        labels = st["labels"]
        scale = st.get("loss_scale", 1.0)
        hits = None if self.env.training else (logits.argmax(-1) == labels).float().mean() * scale
        loss = F.cross_entropy_sum(logits, labels, scale / labels.numel())
        # evaluation: [loss, share of samples whose best class is the label], both averaged the same way downstream
        st["loss"] = loss if hits is None else torch.stack([loss.reshape(()), hits])


class FusedBnAddRelu(FusedGroup):
    """bn3 + residual add (downsample) + relu in ONE normalisation pass."""

    def forward(self, st):
        bn, down = self.members[0], self.members[1]
        x = st["x"]
        r = down.shortcut(st)
        st["x"] = bn.apply(x, residual=r, relu=True)


def fuse_resnet_ops(ops: List[Op]) -> List[Op]:
    out: List[Op] = []
    i = 0
    while i < len(ops):
        if i + 2 < len(ops) and isinstance(ops[i], BNOp) and isinstance(ops[i + 1], DownsampleOp) and \
                isinstance(ops[i + 2], ReLUOp):
            a = ops[i].info
            if all((o.info.tp, o.info.dp, o.info.recompute) == (a.tp, a.dp, a.recompute) for o in ops[i:i + 3]):
                out.append(FusedBnAddRelu(ops[i:i + 3]))
                i += 3
                continue
        if i + 1 < len(ops) and isinstance(ops[i], BNOp) and isinstance(ops[i + 1], ReLUOp) and not ops[i].relu:
            a, b = ops[i].info, ops[i + 1].info
            if (a.tp, a.dp, a.recompute) == (b.tp, b.dp, b.recompute):
                ops[i].relu = True
                grp = FusedGroup(ops[i:i + 2])
                grp.forward = ops[i].forward
                out.append(grp)
                i += 2
                continue
        out.append(ops[i])
        i += 1
    return out


def build_resnet_op(info: OpInfo, env: Env) -> Op:
    c: ResNetConfig = env.cfg
    n = info.name
    if n == "conv1":
        # the stem reads 3 input channels, which cannot be split over a tensor-parallel group: it always splits its
        # output channels, whatever the plan says (the reference's ParallelConvOp, flex_ops.py:1461-1494, would
        # divide 3 by the group size)
        info.algo = 0
        return ConvOp(info, env, 3, c.in_channels, 7, 2, 3)
    if n == "bn1":
        return BNOp(info, env, c.in_channels)
    if n == "relu1":
        return ReLUOp(info, env)
    if n == "maxpool":
        return MaxPoolOp(info, env)
    if n == "avgpool":
        return AvgPoolOp(info, env)
    if n == "fc":
        return FCLossOp(info, env, c.in_channels * 2 ** (len(c.blocks) - 1) * 4, c.num_classes)
    _, g, b, kind = n.split("-")
    g, b = int(g), int(b)
    cin, base, stride, _ = _block_geometry(c, g, b)
    mid, out = base * c.width_factor, base * 4
    if kind == "conv1":
        return ConvOp(info, env, cin, base, 1, 1, 0, keep_residual=True)
    if kind == "bn1":
        return BNOp(info, env, base, relu=c.inner_relu)
    if kind == "conv2":
        return ConvOp(info, env, base, mid, 3, stride, 1)
    if kind == "bn2":
        return BNOp(info, env, mid, relu=c.inner_relu)
    if kind == "conv3":
        return ConvOp(info, env, mid, out, 1, 1, 0)
    if kind == "bn3":
        return BNOp(info, env, out)
    if kind == "downsample":
        return DownsampleOp(info, env, cin, out, stride, project=(b == 0))
    if kind == "relu":
        return ReLUOp(info, env)
    raise KeyError(f"unknown ResNet op {n}")


def resnet_config_from_plan(d: dict, **overrides) -> ResNetConfig:
    cfg = ResNetConfig(blocks=tuple(d["num_layers"]) if isinstance(d["num_layers"], (list, tuple)) else (3, 4, 6, 3),
                       in_channels=d["in_channels"], width_factor=d["width_factor"])
    for k, v in overrides.items():
        setattr(cfg, k, v)
    return cfg
