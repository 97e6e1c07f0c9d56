"""Differentiable ops of the framework: thin autograd wrappers over the sm_100a kernels.

All activations are 2-D ``[tokens, features]`` bf16 matrices with tokens in batch-major order
(``row = b * seq + s``).  Weight gradients are accumulated by the kernels straight into the fp32
``main_grad`` buffer attached to each parameter (gradient-accumulation fusion), so ``backward``
returns ``None`` for parameters that carry a ``main_grad``.

On CUDA tensors the native kernels always run (a missing extension raises).  CPU tensors take a
plain PyTorch implementation of the same math, which is what the multi-process gloo tests and the
numerics oracles use.
"""
from __future__ import annotations

import math
import os

import torch
import torch.nn.functional as F

from . import native

ACT_NONE, ACT_GELU, ACT_RELU, ACT_DGELU, ACT_DRELU = 0, 1, 2, 3, 4
EW_BIAS_GELU, EW_BIAS_GELU_BWD, EW_BIAS_DROP_ADD, EW_DROPOUT, EW_DROPOUT_BWD, EW_RELU, EW_RELU_BWD, EW_ADD = range(8)


# --------------------------------------------------------------------------------------------
# Counter-based seeds for dropout.  Kernels regenerate masks from (seed) alone, so backward and
# activation recompute only need the same seed again: `SeedState` is saved / restored around a
# recomputed segment (the role of the reference's CudaRNGStatesTracker, mpu/random.py:128-197).
# --------------------------------------------------------------------------------------------
class SeedState:
    def __init__(self, base: int = 1234):
        self.base = int(base)
        self.counter = 0

    def next(self) -> int:
        self.counter += 1
        # splitmix-style scramble, kept below 2^62 so it survives the int64 binding
        z = (self.base * 0x9E3779B97F4A7C15 + self.counter * 0xBF58476D1CE4E5B9) & ((1 << 62) - 1)
        return z

    def get_state(self):
        return (self.base, self.counter)

    def set_state(self, st):
        self.base, self.counter = st


_seed_state = SeedState()


def seed_state() -> SeedState:
    return _seed_state


def manual_seed(seed: int) -> None:
    _seed_state.base = int(seed)
    _seed_state.counter = 0


# --------------------------------------------------------------------------------------------
# helpers
# --------------------------------------------------------------------------------------------
def _gelu_tanh(x):
    return 0.5 * x * (1.0 + torch.tanh(0.7978845608028654 * x * (1.0 + 0.044715 * x * x)))


def _gelu_tanh_grad(x):
    t = torch.tanh(0.7978845608028654 * x * (1.0 + 0.044715 * x * x))
    return 0.5 * x * ((1 - t * t) * (0.7978845608028654 + 0.1070322243 * x * x)) + 0.5 * (1 + t)


def _act(x, act):
    if act == ACT_GELU:
        return _gelu_tanh(x)
    if act == ACT_RELU:
        return torch.relu(x)
    return x


def gemm(a, b, out=None, *, a_mn=False, b_mn=False, bias=None, act=ACT_NONE, aux=None, preact_out=None,
         residual=None, accumulate=False, alpha=1.0, dropout_p=0.0, seed=0, out_dtype=torch.bfloat16):
    """Raw GEMM entry (no autograd): out[M,N] = epilogue(alpha * A . B^T), see csrc/gemm_sm100.cuh."""
    M = a.shape[1] if a_mn else a.shape[0]
    N = b.shape[1] if b_mn else b.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    if a.is_cuda:
        native.ext().gemm(a, b, out, a_mn, b_mn, bias, act, aux, preact_out, residual, accumulate, alpha,
                          dropout_p, seed)
        return out
    # CPU restatement (fp32 math)
    A = (a.t() if a_mn else a).float()
    Bm = (b if b_mn else b.t()).float()
    v = alpha * (A @ Bm)
    if bias is not None:
        v = v + bias.float()
    if preact_out is not None:
        preact_out.copy_(v.to(preact_out.dtype))
    if act in (ACT_GELU, ACT_RELU):
        v = _act(v, act)
    elif act == ACT_DGELU:
        v = v * _gelu_tanh_grad(aux.float())
    elif act == ACT_DRELU:
        v = torch.where(aux.float() > 0, v, torch.zeros_like(v))
    assert dropout_p == 0.0, "the CPU restatement has no counter-based dropout"
    if residual is not None:
        v = v + residual.float()
    if accumulate:
        v = v + out.float()
    out.copy_(v.to(out.dtype))
    return out


def _wgrad(param, g2d, x2d):
    """dW[N,K] (+)= g^T x.  Accumulates into param.main_grad when present, else returns the gradient."""
    mg = getattr(param, "main_grad", None)
    if mg is not None:
        gemm(g2d, x2d, out=mg.view(param.shape[0], -1), a_mn=True, b_mn=True, accumulate=True)
        return None
    return gemm(g2d, x2d, a_mn=True, b_mn=True, out_dtype=torch.float32).to(param.dtype)


def _bgrad(param, g2d):
    mg = getattr(param, "main_grad", None)
    if g2d.is_cuda:
        if mg is not None:
            native.ext().colsum(g2d, mg, True)
            return None
        out = torch.empty(g2d.shape[1], dtype=torch.float32, device=g2d.device)
        native.ext().colsum(g2d, out, False)
        return out.to(param.dtype)
    s = g2d.float().sum(0)
    if mg is not None:
        mg.add_(s)
        return None
    return s.to(param.dtype)


def _vec_grad(param, value_fp32):
    mg = getattr(param, "main_grad", None)
    if mg is not None:
        mg.add_(value_fp32.view_as(mg))
        return None
    return value_fp32.to(param.dtype)


def dropout_bwd(g, p, seed):
    if p == 0.0:
        return g
    if g.is_cuda:
        return native.ext().elementwise(EW_DROPOUT_BWD, g.contiguous(), None, None, p, seed)
    raise RuntimeError("counter-based dropout exists only on the GPU path")


# --------------------------------------------------------------------------------------------
# Linear (+ bias + activation + dropout + residual), one GEMM kernel forward, two backward
# --------------------------------------------------------------------------------------------
class LinearFn(torch.autograd.Function):
    """y = residual + dropout(act(x W^T + b)).

    Reference counterparts: ColumnParallelLinear / RowParallelLinear local GEMMs
    (runtime/megatron/mpu/layers.py:282-468) plus the bias-gelu and bias-dropout-add fusions
    (runtime/megatron/model/fused_bias_gelu.py, runtime/megatron/model/flex_ops.py:61-83).
    """

    @staticmethod
    def forward(ctx, x, weight, bias, residual, act, dropout_p, seed):
        need_pre = act in (ACT_GELU, ACT_RELU)
        preact = torch.empty((x.shape[0], weight.shape[0]), dtype=x.dtype, device=x.device) if need_pre else None
        if x.is_cuda or dropout_p == 0.0:
            y = gemm(x, weight, bias=bias, act=act, preact_out=preact, residual=residual, dropout_p=dropout_p,
                     seed=seed)
        else:
            raise RuntimeError("dropout > 0 needs the GPU path")
        ctx.save_for_backward(x, weight, preact)
        ctx.has_bias = bias is not None
        ctx.bias_ref = bias
        ctx.has_res = residual is not None
        ctx.act, ctx.dropout_p, ctx.seed = act, dropout_p, seed
        return y

    @staticmethod
    def backward(ctx, dy):
        x, weight, preact = ctx.saved_tensors
        dy = dy.contiguous()
        dres = dy if ctx.has_res else None
        g = dropout_bwd(dy, ctx.dropout_p, ctx.seed)
        if ctx.act in (ACT_GELU, ACT_RELU):
            op = EW_BIAS_GELU_BWD if ctx.act == ACT_GELU else EW_RELU_BWD
            if g.is_cuda:
                g = native.ext().elementwise(op, preact, g, None, 0.0, 0)
            else:
                pf = preact.float()
                d = _gelu_tanh_grad(pf) if ctx.act == ACT_GELU else (pf > 0).float()
                g = (g.float() * d).to(g.dtype)
        dx = gemm(g, weight, b_mn=True) if ctx.needs_input_grad[0] else None
        dw = _wgrad(weight, g, x) if ctx.needs_input_grad[1] else None
        db = _bgrad(ctx.bias_ref, g) if (ctx.has_bias and ctx.needs_input_grad[2]) else None
        return dx, dw, db, dres, None, None, None


def linear(x, weight, bias=None, residual=None, act=ACT_NONE, dropout_p=0.0, seed=0):
    return LinearFn.apply(x, weight, bias, residual, act, dropout_p, seed)


class RowParallelLinearFusedFn(torch.autograd.Function):
    """y = residual + dropout(all_reduce_tp(x_r W_r^T) + b) with the all-reduce INSIDE the GEMM kernel
    (csrc/gemm_ar_sm100.cu).  Backward needs no collective: dx_r = g W_r, dW_r = g^T x_r with g the masked dy.

    Reference counterpart: RowParallelLinear + reduce_from_tensor_model_parallel_region + bias-dropout-add
    (runtime/megatron/mpu/layers.py:373-468, runtime/megatron/mpu/mappings.py:23-40)."""

    @staticmethod
    def forward(ctx, x, weight, bias, residual, dropout_p, seed, tpctx):
        y = tpctx.linear_allreduce(x, weight, bias=bias, residual=residual, dropout_p=dropout_p, seed=seed)
        ctx.save_for_backward(x, weight)
        ctx.bias_ref = bias
        ctx.has_res = residual is not None
        ctx.dropout_p, ctx.seed = dropout_p, seed
        return y

    @staticmethod
    def backward(ctx, dy):
        x, weight = ctx.saved_tensors
        dy = dy.contiguous()
        dres = dy if ctx.has_res else None
        g = dropout_bwd(dy, ctx.dropout_p, ctx.seed)
        dx = gemm(g, weight, b_mn=True) if ctx.needs_input_grad[0] else None
        dw = _wgrad(weight, g, x) if ctx.needs_input_grad[1] else None
        db = _bgrad(ctx.bias_ref, g) if (ctx.bias_ref is not None and ctx.needs_input_grad[2]) else None
        return dx, dw, db, dres, None, None, None


def row_parallel_linear_fused(x, weight, bias, residual, dropout_p, seed, tpctx):
    return RowParallelLinearFusedFn.apply(x, weight, bias, residual, dropout_p, seed, tpctx)


class ColumnParallelLinearFusedFn(torch.autograd.Function):
    """y_r = act(x W_r^T + b_r) on a replicated input; the backward all-reduce of the input gradient
    (sum over the tp ranks of g_r W_r) runs inside the dgrad GEMM kernel.

    Reference counterpart: copy_to_tensor_model_parallel_region + ColumnParallelLinear
    (runtime/megatron/mpu/layers.py:459-470, runtime/megatron/mpu/mappings.py:79-93)."""

    @staticmethod
    def forward(ctx, x, weight, bias, act, tpctx):
        need_pre = act in (ACT_GELU, ACT_RELU)
        preact = torch.empty((x.shape[0], weight.shape[0]), dtype=x.dtype, device=x.device) if need_pre else None
        y = gemm(x, weight, bias=bias, act=act, preact_out=preact)
        ctx.save_for_backward(x, weight, preact)
        ctx.bias_ref, ctx.act, ctx.tpctx = bias, act, tpctx
        return y

    @staticmethod
    def backward(ctx, dy):
        x, weight, preact = ctx.saved_tensors
        g = dy.contiguous()
        if ctx.act in (ACT_GELU, ACT_RELU):
            op = EW_BIAS_GELU_BWD if ctx.act == ACT_GELU else EW_RELU_BWD
            g = native.ext().elementwise(op, preact, g, None, 0.0, 0)
        dx = ctx.tpctx.linear_allreduce(g, weight, b_mn=True) if ctx.needs_input_grad[0] else None
        dw = _wgrad(weight, g, x) if ctx.needs_input_grad[1] else None
        db = _bgrad(ctx.bias_ref, g) if (ctx.bias_ref is not None and ctx.needs_input_grad[2]) else None
        return dx, dw, db, None, None


def column_parallel_linear_fused(x, weight, bias, act, tpctx):
    return ColumnParallelLinearFusedFn.apply(x, weight, bias, act, tpctx)


class GatheredColumnLinearFn(torch.autograd.Function):
    """y_r = act(concat over the tp ranks of x_s . W_r^T + b_r) for an input whose ROWS are dealt out over the ranks of
    the tensor-parallel group (the previous op ran data parallel over the same GPUs): the gather of the rows runs
    inside the GEMM kernel (csrc/gemm_ag_sm100.cu, csrc/gemm2_sm100.cu), and the backward is the GEMM -> reduce-scatter
    form of the fused GEMM + collective kernel, which leaves on every rank the input gradient of its own rows.

    Reference counterpart: the dp -> tp case of tensor_adapter (all-gather of the rows, backward reduce-scatter;
    runtime/megatron/mpu/mappings.py:382-468, 212-303) followed by ColumnParallelLinear
    (runtime/megatron/mpu/layers.py:459-470)."""

    @staticmethod
    def forward(ctx, x_local, weight, bias, act, tpctx):
        rows, K = x_local.shape
        M = rows * tpctx.tp
        need_pre = act in (ACT_GELU, ACT_RELU)
        preact = torch.empty((M, weight.shape[0]), dtype=x_local.dtype, device=x_local.device) if need_pre else None
        tpctx.ensure_allgather(M, K)
        xl = x_local.contiguous()
        y = tpctx.allgather_linear(xl, weight, bias=bias, act=act, preact_out=preact)
        ctx.save_for_backward(tpctx.gathered_input(xl), weight, preact)
        ctx.bias_ref, ctx.act, ctx.tpctx = bias, act, tpctx
        return y

    @staticmethod
    def backward(ctx, dy):
        x_full, weight, preact = ctx.saved_tensors
        g = dy.contiguous()
        if ctx.act in (ACT_GELU, ACT_RELU):
            op = EW_BIAS_GELU_BWD if ctx.act == ACT_GELU else EW_RELU_BWD
            g = native.ext().elementwise(op, preact, g, None, 0.0, 0)
        # Every rank differentiates the mean loss of ITS rows: going back from the tensor-parallel region (one copy of
        # the rows, data-parallel degree 1) to the ranks that hold tp disjoint row shares, the gradient is scaled by
        # tp, so that the 1 / dp averaging of the parameter gradients upstream still yields the global mean (the
        # relayout engine applies the same factor, parallel/relayout.py::plan_transfer)
        dx = (ctx.tpctx.linear_reduce_scatter(g, weight, b_mn=True, alpha=float(ctx.tpctx.tp))
              if ctx.needs_input_grad[0] else None)
        dw = _wgrad(weight, g, x_full) if ctx.needs_input_grad[1] else None
        db = _bgrad(ctx.bias_ref, g) if (ctx.bias_ref is not None and ctx.needs_input_grad[2]) else None
        return dx, dw, db, None, None


def gathered_column_linear_fused(x_local, weight, bias, act, tpctx):
    return GatheredColumnLinearFn.apply(x_local, weight, bias, act, tpctx)


def can_gather_in_gemm(x_local, tpctx) -> bool:
    """Shapes the fused all-gather -> GEMM and GEMM -> reduce-scatter kernels take: whole 128-row blocks per rank, a
    reduction length in whole 64-column tiles, and a fused scratch that holds the gathered product."""
    if tpctx is None or x_local.dim() != 2 or not x_local.is_cuda:
        return False
    rows, K = x_local.shape
    return rows % 128 == 0 and K % 64 == 0 and tpctx.fits(rows * tpctx.tp, K)


class MLPFn(torch.autograd.Function):
    """y = residual + dropout(act(x W1^T + b1) W2^T + b2) with the activation derivative folded into the
    dgrad GEMM epilogue of the second layer (4 ops of the reference op list in 2 forward / 4 backward GEMMs:
    MLP-GEMM-1, MLP-gelu, MLP-GEMM-2, post-MLP-dropout; runtime/megatron/model/flex_gpt.py:18-41)."""

    @staticmethod
    def forward(ctx, x, w1, b1, w2, b2, residual, act, dropout_p, seed):
        pre = torch.empty((x.shape[0], w1.shape[0]), dtype=x.dtype, device=x.device)
        h = gemm(x, w1, bias=b1, act=act, preact_out=pre)
        y = gemm(h, w2, bias=b2, residual=residual, dropout_p=dropout_p, seed=seed)
        ctx.save_for_backward(x, w1, w2, pre, h)
        ctx.b1, ctx.b2 = b1, b2
        ctx.has_res = residual is not None
        ctx.act, ctx.dropout_p, ctx.seed = act, dropout_p, seed
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w1, w2, pre, h = ctx.saved_tensors
        dy = dy.contiguous()
        dres = dy if ctx.has_res else None
        g2 = dropout_bwd(dy, ctx.dropout_p, ctx.seed)
        dw2 = _wgrad(w2, g2, h)
        db2 = _bgrad(ctx.b2, g2) if ctx.b2 is not None else None
        dact = ACT_DGELU if ctx.act == ACT_GELU else ACT_DRELU
        g1 = gemm(g2, w2, b_mn=True, act=dact, aux=pre)
        dw1 = _wgrad(w1, g1, x)
        db1 = _bgrad(ctx.b1, g1) if ctx.b1 is not None else None
        dx = gemm(g1, w1, b_mn=True) if ctx.needs_input_grad[0] else None
        return dx, dw1, db1, dw2, db2, dres, None, None, None


def mlp(x, w1, b1, w2, b2, residual=None, act=ACT_GELU, dropout_p=0.0, seed=0):
    return MLPFn.apply(x, w1, b1, w2, b2, residual, act, dropout_p, seed)


# --------------------------------------------------------------------------------------------
# LayerNorm
# --------------------------------------------------------------------------------------------
class LayerNormFn(torch.autograd.Function):
    """LayerNorm over the last dim with fp32 gamma / beta (reference: fused_layer_norm.py MixedFusedLayerNorm
    over runtime/megatron/fused_kernels/layer_norm_cuda_kernel.cu).

    With `pass_through` the function also returns its input as a second output, for the residual branch that
    skips the normalised sub-layer: the gradients of both branches then arrive together and the backward kernel adds
    the residual branch's while it writes dx (instead of autograd adding two [tokens, hidden] tensors afterwards)."""

    @staticmethod
    def forward(ctx, x, gamma, beta, eps, pass_through):
        if x.is_cuda:
            y, mean, rstd = native.ext().layernorm_fwd(x, None, gamma, beta, eps)
        else:
            xf = x.float()
            mean = xf.mean(-1)
            var = xf.var(-1, unbiased=False)
            rstd = torch.rsqrt(var + eps)
            y = ((xf - mean[:, None]) * rstd[:, None] * gamma.float() + beta.float()).to(x.dtype)
        ctx.save_for_backward(x, gamma, mean, rstd)
        ctx.params = (gamma, beta)
        ctx.set_materialize_grads(False)
        if pass_through:
            return y, x.view_as(x)
        return y

    @staticmethod
    def backward(ctx, dy, dres=None):
        x, gamma, mean, rstd = ctx.saved_tensors
        g_param, b_param = ctx.params
        if dy is None:                      # only the residual branch was used
            return dres, None, None, None, None
        dy = dy.contiguous()
        if dres is not None:
            dres = dres.contiguous()
        mg_g, mg_b = getattr(g_param, "main_grad", None), getattr(b_param, "main_grad", None)
        if x.is_cuda:
            if mg_g is not None and mg_b is not None:
                dx = native.ext().layernorm_bwd(dy, x, gamma, mean, rstd, dres, mg_g, mg_b, True)
                return dx, None, None, None, None
            dg = torch.empty_like(gamma, dtype=torch.float32)
            db = torch.empty_like(gamma, dtype=torch.float32)
            dx = native.ext().layernorm_bwd(dy, x, gamma, mean, rstd, dres, dg, db, False)
            return dx, dg.to(gamma.dtype), db.to(gamma.dtype), None, None
        xf, dyf = x.float(), dy.float()
        xhat = (xf - mean[:, None]) * rstd[:, None]
        dg = (dyf * xhat).sum(0)
        db = dyf.sum(0)
        dxhat = dyf * gamma.float()
        dx = rstd[:, None] * (dxhat - dxhat.mean(-1, keepdim=True) - xhat * (dxhat * xhat).mean(-1, keepdim=True))
        if dres is not None:
            dx = dx + dres.float()
        return dx.to(x.dtype), _vec_grad(g_param, dg), _vec_grad(b_param, db), None, None


def layernorm(x, gamma, beta, eps=1e-5):
    return LayerNormFn.apply(x, gamma, beta, eps, False)


def layernorm_keep_input(x, gamma, beta, eps=1e-5):
    """(LayerNorm(x), x): the second value is x for the residual add behind the normalised sub-layer."""
    return LayerNormFn.apply(x, gamma, beta, eps, True)


# --------------------------------------------------------------------------------------------
# Elementwise ops that can stand alone in a stage
# --------------------------------------------------------------------------------------------
class BiasActFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, bias, act):
        ctx.save_for_backward(x)
        ctx.bias, ctx.act = bias, act
        if x.is_cuda:
            return native.ext().elementwise(EW_BIAS_GELU if act == ACT_GELU else EW_RELU, x.contiguous(), None, bias,
                                            0.0, 0)
        v = x.float() + (bias.float() if bias is not None else 0.0)
        return _act(v, act).to(x.dtype)

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        dy = dy.contiguous()
        if x.is_cuda:
            g = native.ext().elementwise(EW_BIAS_GELU_BWD if ctx.act == ACT_GELU else EW_RELU_BWD, x.contiguous(), dy,
                                         ctx.bias, 0.0, 0)
        else:
            v = x.float() + (ctx.bias.float() if ctx.bias is not None else 0.0)
            d = _gelu_tanh_grad(v) if ctx.act == ACT_GELU else (v > 0).float()
            g = (dy.float() * d).to(dy.dtype)
        db = _bgrad(ctx.bias, g) if ctx.bias is not None else None
        return g, db, None


def bias_act(x, bias, act=ACT_GELU):
    return BiasActFn.apply(x, bias, act)


class BiasDropoutAddFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, bias, residual, p, seed):
        ctx.bias, ctx.p, ctx.seed = bias, p, seed
        if x.is_cuda:
            return native.ext().elementwise(EW_BIAS_DROP_ADD, x.contiguous(), residual.contiguous(), bias, p, seed)
        assert p == 0.0, "dropout > 0 needs the GPU path"
        return (x.float() + (bias.float() if bias is not None else 0.0) + residual.float()).to(x.dtype)

    @staticmethod
    def backward(ctx, dy):
        dy = dy.contiguous()
        g = dropout_bwd(dy, ctx.p, ctx.seed)
        db = _bgrad(ctx.bias, g) if ctx.bias is not None else None
        return g, db, dy, None, None


def bias_dropout_add(x, bias, residual, p=0.0, seed=0):
    return BiasDropoutAddFn.apply(x, bias, residual, p, seed)


class DropoutFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, p, seed):
        ctx.p, ctx.seed = p, seed
        if p == 0.0:
            return x
        if x.is_cuda:
            return native.ext().elementwise(EW_DROPOUT, x.contiguous(), None, None, p, seed)
        raise RuntimeError("dropout > 0 needs the GPU path")

    @staticmethod
    def backward(ctx, dy):
        return dropout_bwd(dy.contiguous(), ctx.p, ctx.seed), None, None


def dropout(x, p, seed):
    return DropoutFn.apply(x, p, seed)


# --------------------------------------------------------------------------------------------
# Attention
# --------------------------------------------------------------------------------------------
def _attn_reference(q, k, v, B, NH, SQ, SK, HD, scale, causal, kv_lens):
    qf = q.float().view(B, SQ, NH, HD).transpose(1, 2)
    kf = k.float().view(B, SK, NH, HD).transpose(1, 2)
    vf = v.float().view(B, SK, NH, HD).transpose(1, 2)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if causal:
        mask = torch.ones(SQ, SK, dtype=torch.bool, device=q.device).tril()
        s = s.masked_fill(~mask, float("-inf"))
    if kv_lens is not None:
        idx = torch.arange(SK, device=q.device)[None, None, None, :]
        s = s.masked_fill(idx >= kv_lens.view(B, 1, 1, 1), float("-inf"))
    p = torch.softmax(s, dim=-1)
    o = torch.matmul(p, vf)
    return o.transpose(1, 2).reshape(B * SQ, NH * HD)


class FlashAttnFn(torch.autograd.Function):
    """softmax(scale * Q K^T [+ causal / key-length mask]) V with dropout on the probabilities.

    q, k, v are 2-D matrices [B*S, ld]; head h occupies columns [col0 + h*HD, col0 + (h+1)*HD), which lets
    the three operands be column ranges of one QKV GEMM output (no split / transpose copies).
    Stands for score + softmax + dropout + context of the reference
    (runtime/megatron/model/flex_ops.py:711-1015)."""

    @staticmethod
    def forward(ctx, q, k, v, B, NH, SQ, SK, HD, cols, scale, causal, kv_lens, dropout_p, seed, bias_table=None):
        qc, kc, vc = cols
        ctx.has_bias = bias_table is not None
        if q.is_cuda:
            bt = bias_table.float().contiguous() if bias_table is not None else None
            o, lse = native.ext().attn_fwd(q, k, v, B, NH, SQ, SK, HD, qc, kc, vc, scale, causal, kv_lens, dropout_p,
                                           seed, bt)
            ctx.save_for_backward(q, k, v, o, lse, kv_lens if kv_lens is not None else torch.empty(0),
                                  bt if bt is not None else torch.empty(0))
        else:
            assert bias_table is None, "the score bias exists on the GPU path and in attention_with_bias"
            assert dropout_p == 0.0, "dropout > 0 needs the GPU path"
            w = NH * HD
            o = _attn_reference(q[:, qc:qc + w], k[:, kc:kc + w], v[:, vc:vc + w], B, NH, SQ, SK, HD, scale, causal,
                                kv_lens).to(q.dtype)
            ctx.save_for_backward(q, k, v, o, torch.empty(0), kv_lens if kv_lens is not None else torch.empty(0),
                                  torch.empty(0))
        ctx.dims = (B, NH, SQ, SK, HD)
        ctx.cols, ctx.scale, ctx.causal, ctx.dropout_p, ctx.seed = cols, scale, causal, dropout_p, seed
        ctx.has_lens = kv_lens is not None
        ctx.same_qkv = (q.data_ptr() == k.data_ptr() == v.data_ptr()) and q.shape == k.shape == v.shape
        ctx.same_kv = (k.data_ptr() == v.data_ptr()) and k.shape == v.shape
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse, kv_lens, bias_table = ctx.saved_tensors
        kv_lens = kv_lens if ctx.has_lens else None
        bias_table = bias_table if ctx.has_bias else None
        dbias = torch.zeros_like(bias_table) if bias_table is not None else None
        B, NH, SQ, SK, HD = ctx.dims
        qc, kc, vc = ctx.cols
        do = do.contiguous()
        if q.is_cuda:
            # gradients land in matrices laid out like their inputs, so a fused QKV input gets ONE gradient;
            # columns no head writes (a wider carrier matrix) must read as zero
            w = NH * HD

            def _grad_like(t, heads_cols):
                return torch.empty_like(t) if t.shape[1] == heads_cols else torch.zeros_like(t)

            if ctx.same_qkv:
                dq = _grad_like(q, 3 * w)
                dk = dv = dq
            elif ctx.same_kv:
                dq = _grad_like(q, w)
                dk = _grad_like(k, 2 * w)
                dv = dk
            else:
                dq, dk, dv = _grad_like(q, w), _grad_like(k, w), _grad_like(v, w)
            native.ext().attn_bwd(q, k, v, o, lse, do, dq, dk, dv, B, NH, SQ, SK, HD, qc, kc, vc, qc, kc, vc,
                                  ctx.scale, ctx.causal, kv_lens, ctx.dropout_p, ctx.seed, bias_table, dbias)
            if ctx.same_qkv:
                return (dq, None, None) + (None,) * 11 + (dbias,)
            if ctx.same_kv:
                return (dq, dk, None) + (None,) * 11 + (dbias,)
            return (dq, dk, dv) + (None,) * 11 + (dbias,)
        w = NH * HD
        with torch.enable_grad():
            qq = q[:, qc:qc + w].detach().float().requires_grad_(True)
            kk = k[:, kc:kc + w].detach().float().requires_grad_(True)
            vv = v[:, vc:vc + w].detach().float().requires_grad_(True)
            oo = _attn_reference(qq, kk, vv, B, NH, SQ, SK, HD, ctx.scale, ctx.causal, kv_lens)
            gq, gk, gv = torch.autograd.grad(oo, (qq, kk, vv), do.float())
        dq = torch.zeros_like(q)
        dq[:, qc:qc + w] = gq.to(q.dtype)
        if ctx.same_qkv:
            dq[:, kc:kc + w] = gk.to(q.dtype)
            dq[:, vc:vc + w] = gv.to(q.dtype)
            return (dq, None, None) + (None,) * 12
        dk = torch.zeros_like(k)
        dk[:, kc:kc + w] = gk.to(k.dtype)
        if ctx.same_kv:
            dk[:, vc:vc + w] = gv.to(k.dtype)
            return (dq, dk, None) + (None,) * 12
        dv = torch.zeros_like(v)
        dv[:, vc:vc + w] = gv.to(v.dtype)
        return (dq, dk, dv) + (None,) * 12


def flash_attention(q, k, v, B, NH, SQ, SK, HD, cols=(0, 0, 0), scale=None, causal=False, kv_lens=None,
                    dropout_p=0.0, seed=0, bias_table=None):
    """bias_table (GPU path): fp32 [NH, SQ + SK - 1], differentiable; the scores of head h get
    bias_table[h, key - query + SQ - 1] added after the scale (a relative-position bias as a table over the distance)."""
    if scale is None:
        scale = 1.0 / math.sqrt(HD)
    return FlashAttnFn.apply(q, k, v, B, NH, SQ, SK, HD, tuple(cols), float(scale), bool(causal), kv_lens,
                             float(dropout_p), int(seed), bias_table)


def attention_with_bias(qkv, B, NH, S, HD, scale, causal, kv_lens, bias, dropout_p=0.0):
    """Self-attention on a fused QKV matrix with an additive [NH, S, S] bias on the scores: plain differentiable
    PyTorch (fp32), the reference for kernels that take the bias as a per-head distance table."""
    assert dropout_p == 0.0, "dropout > 0 needs the GPU path"
    w = NH * HD
    q = qkv[:, :w].float().view(B, S, NH, HD).transpose(1, 2)
    k = qkv[:, w:2 * w].float().view(B, S, NH, HD).transpose(1, 2)
    v = qkv[:, 2 * w:3 * w].float().view(B, S, NH, HD).transpose(1, 2)
    s = torch.matmul(q, k.transpose(-1, -2)) * scale + bias[None].float()
    if causal:
        s = s.masked_fill(~torch.ones(S, S, dtype=torch.bool, device=qkv.device).tril(), float("-inf"))
    if kv_lens is not None:
        idx = torch.arange(S, device=qkv.device)[None, None, None, :]
        s = s.masked_fill(idx >= kv_lens.view(B, 1, 1, 1), float("-inf"))
    o = torch.matmul(torch.softmax(s, dim=-1), v)
    return o.transpose(1, 2).reshape(B * S, w).to(qkv.dtype)


def fused_qkv_attention(qkv, B, NH, S, HD, causal=True, dropout_p=0.0, seed=0, scale=None):
    """Self-attention on a fused QKV matrix [B*S, 3*NH*HD] laid out as [Q heads | K heads | V heads]."""
    h = NH * HD
    return flash_attention(qkv, qkv, qkv, B, NH, S, S, HD, cols=(0, h, 2 * h), scale=scale, causal=causal,
                           dropout_p=dropout_p, seed=seed)


# --------------------------------------------------------------------------------------------
# Stand-alone softmax (unfused attention fallback)
# --------------------------------------------------------------------------------------------
class ScaledSoftmaxFn(torch.autograd.Function):
    """mode 0 plain / 1 causal / 2 masked scaled softmax over the last dim of [b, np, sq, sk]
    (reference: runtime/megatron/model/fused_softmax.py over the three softmax extensions)."""

    @staticmethod
    def forward(ctx, x, mask, scale, mode):
        if x.is_cuda:
            y = native.ext().softmax_fwd(x.contiguous(), mask, scale, mode, x.shape[-3] if x.dim() >= 3 else 1)
        else:
            s = x.float() * scale
            if mode == 1:
                sq, sk = s.shape[-2:]
                s = s.masked_fill(~torch.ones(sq, sk, dtype=torch.bool).tril(), float("-inf"))
            elif mode == 2:
                s = s.masked_fill(mask.bool(), -10000.0)
            y = torch.softmax(s, -1).to(x.dtype)
        ctx.save_for_backward(y)
        ctx.scale = scale
        return y

    @staticmethod
    def backward(ctx, g):
        (y,) = ctx.saved_tensors
        if y.is_cuda:
            return native.ext().softmax_bwd(g.contiguous(), y, ctx.scale), None, None, None
        yf, gf = y.float(), g.float()
        dx = ctx.scale * (gf * yf - yf * (gf * yf).sum(-1, keepdim=True))
        return dx.to(y.dtype), None, None, None


def scaled_softmax(x, scale=1.0, mode=0, mask=None):
    return ScaledSoftmaxFn.apply(x, mask, float(scale), int(mode))


# --------------------------------------------------------------------------------------------
# Embedding and LM head + cross entropy
# --------------------------------------------------------------------------------------------
_DETERMINISTIC_EMBEDDING_GRAD = [os.environ.get("SSB_EMBEDDING_GRAD_ATOMICS", "0") != "1"]


class EmbeddingFn(torch.autograd.Function):
    """dropout(W[ids - v0] (0 outside the local vocab range) + P[pos]).  Vocab-parallel ranks all-reduce the
    result outside (reference: runtime/megatron/mpu/layers.py:136-205, flex_ops.py:229-380)."""

    @staticmethod
    def forward(ctx, ids, pos, W, P, v0, dropout_p, seed):
        ctx.args = (v0, dropout_p, seed)
        ctx.params = (W, P)
        ctx.save_for_backward(ids, pos if pos is not None else torch.empty(0))
        ctx.has_pos = pos is not None
        if W.is_cuda:
            return native.ext().embedding_fwd(ids.contiguous().view(-1), pos.contiguous().view(-1) if pos is not None
                                              else None, W, P, v0, dropout_p, seed)
        assert dropout_p == 0.0, "dropout > 0 needs the GPU path"
        flat = ids.reshape(-1)
        local = (flat >= v0) & (flat < v0 + W.shape[0])
        out = torch.where(local[:, None], W.float()[(flat - v0).clamp(0, W.shape[0] - 1)], torch.zeros(1))
        if P is not None:
            out = out + P.float()[pos.view(-1)]
        return out.to(W.dtype)

    @staticmethod
    def backward(ctx, g):
        ids, pos = ctx.saved_tensors
        pos = pos if ctx.has_pos else None
        W, P = ctx.params
        v0, dropout_p, seed = ctx.args
        g = g.contiguous()
        mgW = getattr(W, "main_grad", None)
        mgP = getattr(P, "main_grad", None) if P is not None else None
        if g.is_cuda:
            dW = mgW if mgW is not None else torch.zeros(W.shape, dtype=torch.float32, device=g.device)
            dP = None
            if P is not None:
                dP = mgP if mgP is not None else torch.zeros(P.shape, dtype=torch.float32, device=g.device)
            if _DETERMINISTIC_EMBEDDING_GRAD[0]:
                # rows are summed run by run in token order: repeated runs give bitwise equal gradients
                for keys_t, dst, k0 in ((ids, dW, v0), (pos, dP, 0)):
                    if keys_t is not None and dst is not None:
                        keys, order = torch.sort(keys_t.contiguous().view(-1), stable=True)
                        native.ext().embedding_bwd_sorted(keys, order, g, dst, k0, dropout_p, seed)
            else:
                native.ext().embedding_bwd(ids.contiguous().view(-1), pos.contiguous().view(-1) if pos is not None
                                           else None, g, dW, dP, v0, dropout_p, seed)
            return (None, None, None if mgW is not None else dW.to(W.dtype),
                    None if (P is None or mgP is not None) else dP.to(P.dtype), None, None, None)
        flat = ids.view(-1)
        local = (flat >= v0) & (flat < v0 + W.shape[0])
        dW = torch.zeros(W.shape, dtype=torch.float32)
        dW.index_add_(0, (flat - v0)[local], g.float()[local])
        dP = None
        if P is not None:
            dP = torch.zeros(P.shape, dtype=torch.float32)
            dP.index_add_(0, pos.view(-1), g.float())
        return (None, None, _vec_grad(W, dW), _vec_grad(P, dP) if P is not None else None, None, None, None)


def set_deterministic_embedding_grad(on: bool) -> None:
    """Selects how the embedding gradient is scattered on the GPU: sorted runs with plain stores (order
    independent, the default) or float atomics (order dependent in the last bit)."""
    _DETERMINISTIC_EMBEDDING_GRAD[0] = bool(on)


def set_deterministic(on: bool) -> None:
    """Bitwise-reproducible training steps on the GPU.  On: the embedding gradient is summed in sorted runs (the
    default anyway) and the attention backward runs as the dK/dV + dQ kernel pair.  Off (the default for attention):
    the fused attention backward kernel, which sums the key blocks' shares of dQ in an fp32 buffer in the order
    they arrive, so dQ may differ in the last bit between two runs of the same step."""
    set_deterministic_embedding_grad(on)
    if native.available():
        native.ext().set_attn_bwd_deterministic(bool(on))


def embedding(ids, pos, W, P=None, v0=0, dropout_p=0.0, seed=0):
    return EmbeddingFn.apply(ids, pos, W, P, v0, dropout_p, seed)


class LMHeadCrossEntropyFn(torch.autograd.Function):
    """loss_sum = sum_rows mask * CE(x W^T, target) * loss_scale, with W [V_local, H] (tied embedding).

    The logits are produced by the GEMM kernel in bf16, reduced to per-row statistics, (all-reduced across
    the tensor-parallel group when `group` is given), and overwritten in place by their gradient, so the
    backward pass is two more GEMMs and no pass over the logits
    (reference: runtime/megatron/model/language_model.py:24-39 + runtime/megatron/mpu/cross_entropy.py:36-115).
    The op must be the last one of the graph: backward ignores the incoming gradient value (taken as 1)."""

    @staticmethod
    def forward(ctx, x, W, targets, loss_mask, v0, loss_scale, group):
        logits = gemm(x, W)
        tflat = targets.contiguous().view(-1)
        if x.is_cuda:
            st = native.ext().ce_stats(logits, tflat, v0)
            if group is not None and torch.distributed.get_world_size(group) > 1:
                gmax = st[0].clone()
                torch.distributed.all_reduce(gmax, op=torch.distributed.ReduceOp.MAX, group=group)
                st[1].mul_(torch.exp(st[0] - gmax))
                st[0].copy_(gmax)
                torch.distributed.all_reduce(st[1:], group=group)
            losses = native.ext().ce_finalize(logits, tflat, st, loss_mask, v0, loss_scale, True)
            loss = losses.sum() * loss_scale
            dlogits = logits
        else:
            lf = logits.float()
            V = W.shape[0]
            lmax = lf.max(-1).values
            if group is not None and torch.distributed.get_world_size(group) > 1:
                torch.distributed.all_reduce(lmax, op=torch.distributed.ReduceOp.MAX, group=group)
            ex = torch.exp(lf - lmax[:, None])
            ssum = ex.sum(-1)
            local = (tflat >= v0) & (tflat < v0 + V)
            tl = torch.where(local, lf.gather(1, (tflat - v0).clamp(0, V - 1)[:, None])[:, 0], torch.zeros(1))
            if group is not None and torch.distributed.get_world_size(group) > 1:
                torch.distributed.all_reduce(ssum, group=group)
                torch.distributed.all_reduce(tl, group=group)
            w = loss_mask.float().view(-1) if loss_mask is not None else torch.ones_like(ssum)
            losses = (torch.log(ssum) + lmax - tl) * w
            loss = losses.sum() * loss_scale
            prob = ex / ssum[:, None]
            onehot = torch.zeros_like(prob)
            onehot[local, (tflat - v0)[local]] = 1.0
            dlogits = ((prob - onehot) * (w * loss_scale)[:, None]).to(x.dtype)
        ctx.save_for_backward(x, W, dlogits)
        return loss

    @staticmethod
    def backward(ctx, gl):
        x, W, dlogits = ctx.saved_tensors
        dx = gemm(dlogits, W, b_mn=True) if ctx.needs_input_grad[0] else None
        dw = _wgrad(W, dlogits, x) if ctx.needs_input_grad[1] else None
        return dx, dw, None, None, None, None, None


def lm_head_cross_entropy(x, W, targets, loss_mask=None, v0=0, loss_scale=1.0, group=None):
    return LMHeadCrossEntropyFn.apply(x, W, targets, loss_mask, v0, float(loss_scale), group)


class CrossEntropyFn(torch.autograd.Function):
    """sum_rows CE(logits, target) * loss_scale on given logits (used by classifiers whose head has a bias).
    Must be the last op of the graph: backward ignores the incoming gradient value (taken as 1)."""

    @staticmethod
    def forward(ctx, logits, targets, loss_scale):
        tflat = targets.contiguous().view(-1)
        if logits.is_cuda:
            work = logits.contiguous().clone()
            st = native.ext().ce_stats(work, tflat, 0)
            losses = native.ext().ce_finalize(work, tflat, st, None, 0, loss_scale, True)
            ctx.save_for_backward(work)
            return losses.sum() * loss_scale
        lf = logits.float()
        losses = F.cross_entropy(lf, tflat, reduction="none")
        prob = torch.softmax(lf, -1)
        prob[torch.arange(lf.shape[0]), tflat] -= 1.0
        ctx.save_for_backward((prob * loss_scale).to(logits.dtype))
        return losses.sum() * loss_scale

    @staticmethod
    def backward(ctx, g):
        (dlogits,) = ctx.saved_tensors
        return dlogits, None, None


def cross_entropy_sum(logits, targets, loss_scale=1.0):
    return CrossEntropyFn.apply(logits, targets, float(loss_scale))
