"""Differentiable convolution / BatchNorm / pooling ops for NHWC bf16 activations.

A convolution is a GEMM on the tcgen05 kernel: directly on the activation for 1x1 filters, on the patch matrix
written by the im2col kernel for k x k filters (weights are stored [Cout, kh*kw*Cin], tap-major).  CPU tensors take
plain PyTorch restatements (used by the oracles and the gloo tests).
Reference counterparts: ParallelConvOp, ParallelBatchNormOp, ParallelMaxPoolOp, ParallelAdapAvgPoolOp
(runtime/megatron/model/flex_ops.py:1423-1719).
"""
from __future__ import annotations

import torch
import torch.nn.functional as TF

from . import native
from .functional import _vec_grad, _wgrad, gemm


def _pad8(n: int) -> int:
    return (n + 7) // 8 * 8


class Conv2dFn(torch.autograd.Function):
    """y[N,Ho,Wo,Cout] = conv(x[N,H,W,Cin], w[Cout, Kpad]) with Kpad = pad8(kh*kw*Cin), no bias."""

    @staticmethod
    def forward(ctx, x, w, kh, kw, stride, pad):
        N, H, W, C = x.shape
        Ho, Wo = (H + 2 * pad - kh) // stride + 1, (W + 2 * pad - kw) // stride + 1
        ctx.geom = (N, H, W, C, kh, kw, stride, pad, Ho, Wo)
        if not x.is_cuda:
            w4 = w[:, :kh * kw * C].float().view(-1, kh, kw, C).permute(0, 3, 1, 2)
            y = TF.conv2d(x.float().permute(0, 3, 1, 2), w4, stride=stride, padding=pad).permute(0, 2, 3, 1)
            ctx.save_for_backward(x, w)
            return y.contiguous().to(x.dtype)
        ext = native.ext()
        if kh == 1 and kw == 1:
            xs = x if stride == 1 else ext.subsample(x.contiguous(), H, W, stride, False)
            a = xs.reshape(-1, C)
        else:
            a = ext.im2col(x.contiguous(), kh, kw, stride, pad, w.shape[1])
        y = gemm(a, w)
        ctx.save_for_backward(a, w)
        return y.view(N, Ho, Wo, -1)

    @staticmethod
    def backward(ctx, dy):
        N, H, W, C, kh, kw, stride, pad, Ho, Wo = ctx.geom
        a, w = ctx.saved_tensors
        if not dy.is_cuda:
            x = a
            with torch.enable_grad():
                xx = x.detach().float().requires_grad_(True)
                ww = w.detach().float().requires_grad_(True)
                w4 = ww[:, :kh * kw * C].view(-1, kh, kw, C).permute(0, 3, 1, 2)
                y = TF.conv2d(xx.permute(0, 3, 1, 2), w4, stride=stride, padding=pad).permute(0, 2, 3, 1)
                gx, gw = torch.autograd.grad(y, (xx, ww), dy.float())
            return gx.to(x.dtype), _vec_grad(w, gw), None, None, None, None
        ext = native.ext()
        g = dy.reshape(-1, dy.shape[-1]).contiguous()
        dw = _wgrad(w, g, a) if ctx.needs_input_grad[1] else None
        dx = None
        if ctx.needs_input_grad[0]:
            da = gemm(g, w, b_mn=True)                      # [N*Ho*Wo, Kpad]
            if kh == 1 and kw == 1:
                da = da.view(N, Ho, Wo, C)
                dx = da if stride == 1 else ext.subsample(da, H, W, stride, True)
            else:
                dx = ext.col2im(da, N, H, W, C, kh, kw, stride, pad)
        return dx, dw, None, None, None, None


def conv2d(x, w, kh, kw, stride=1, pad=0):
    return Conv2dFn.apply(x, w, kh, kw, stride, pad)


class BatchNormFn(torch.autograd.Function):
    """y = [relu](BN(x) [+ residual]) over the rows of x viewed as [N*H*W, C], batch statistics, fp32 gamma / beta."""

    @staticmethod
    def forward(ctx, x, residual, gamma, beta, run_mean, run_var, eps, momentum, relu):
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        r2 = residual.reshape(-1, shape[-1]).contiguous() if residual is not None else None
        if x.is_cuda:
            y, mean, rstd = native.ext().bn_fwd(x2.contiguous(), r2, gamma, beta, run_mean, run_var, eps, momentum, relu)
        else:
            xf = x2.float()
            mean = xf.mean(0)
            var = xf.var(0, unbiased=False)
            rstd = torch.rsqrt(var + eps)
            if run_mean is not None:
                # same update as the kernel (and torch.nn.BatchNorm2d): unbiased variance into the running estimate
                n = xf.shape[0]
                run_mean.mul_(1.0 - momentum).add_(mean, alpha=momentum)
                run_var.mul_(1.0 - momentum).add_(var * (n / max(n - 1, 1)), alpha=momentum)
            y = (xf - mean) * rstd * gamma.float() + beta.float()
            if r2 is not None:
                y = y + r2.float()
            if relu:
                y = torch.relu(y)
            y = y.to(x.dtype)
        ctx.save_for_backward(x2, y, mean, rstd, gamma)
        ctx.params = (gamma, beta)
        ctx.relu, ctx.has_res, ctx.shape = relu, residual is not None, shape
        return y.view(shape)

    @staticmethod
    def backward(ctx, dy):
        x2, y, mean, rstd, gamma = ctx.saved_tensors
        g_param, b_param = ctx.params
        dy2 = dy.reshape(-1, ctx.shape[-1]).contiguous()
        if dy.is_cuda:
            mg_g, mg_b = getattr(g_param, "main_grad", None), getattr(b_param, "main_grad", None)
            acc = mg_g is not None and mg_b is not None
            dg = mg_g if acc else torch.empty_like(gamma, dtype=torch.float32)
            db = mg_b if acc else torch.empty_like(gamma, dtype=torch.float32)
            outs = native.ext().bn_bwd(dy2, x2, y, mean, rstd, gamma, dg, db, acc, ctx.relu, ctx.has_res)
            dx = outs[0].view(ctx.shape)
            dres = outs[1].view(ctx.shape) if ctx.has_res else None
            return (dx, dres, None if acc else dg.to(gamma.dtype), None if acc else db.to(gamma.dtype),
                    None, None, None, None, None)
        g = dy2.float()
        if ctx.relu:
            g = g * (y.float() > 0)
        xhat = (x2.float() - mean) * rstd
        dgam, dbet = (g * xhat).sum(0), g.sum(0)
        n = x2.shape[0]
        dx = gamma.float() * rstd * (g - dbet / n - xhat * dgam / n)
        return (dx.to(x2.dtype).view(ctx.shape), g.to(x2.dtype).view(ctx.shape) if ctx.has_res else None,
                _vec_grad(g_param, dgam), _vec_grad(b_param, dbet), None, None, None, None, None)


def batch_norm(x, gamma, beta, residual=None, run_mean=None, run_var=None, eps=1e-5, momentum=0.1, relu=False):
    return BatchNormFn.apply(x, residual, gamma, beta, run_mean, run_var, eps, momentum, relu)


@torch.no_grad()
def batch_norm_inference(x, gamma, beta, run_mean, run_var, residual=None, eps=1e-5, relu=False):
    """Evaluation-mode BatchNorm as torch.nn.BatchNorm2d.eval(): normalises with the running estimates and leaves
    them untouched (the reference evaluates with torch's module, runtime/megatron/model/flex_ops.py:1561-1600)."""
    shape = x.shape
    x2 = x.reshape(-1, shape[-1])
    r2 = residual.reshape(-1, shape[-1]).contiguous() if residual is not None else None
    rstd = torch.rsqrt(run_var.float() + eps)
    if x.is_cuda:
        y = native.ext().bn_apply(x2.contiguous(), r2, run_mean, rstd, gamma, beta, relu)
    else:
        y = (x2.float() - run_mean) * rstd * gamma.float() + beta.float()
        if r2 is not None:
            y = y + r2.float()
        if relu:
            y = torch.relu(y)
        y = y.to(x.dtype)
    return y.view(shape)


class MaxPool3x3s2Fn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        ctx.hw = (x.shape[1], x.shape[2])
        if x.is_cuda:
            y, idx = native.ext().maxpool_fwd(x.contiguous())
            ctx.save_for_backward(idx)
            return y
        xf = x.float().permute(0, 3, 1, 2)
        y, idx = TF.max_pool2d(xf, 3, 2, 1, return_indices=True)
        ctx.save_for_backward(idx)
        ctx.cpu_shape = xf.shape
        return y.permute(0, 2, 3, 1).contiguous().to(x.dtype)

    @staticmethod
    def backward(ctx, dy):
        (idx,) = ctx.saved_tensors
        H, W = ctx.hw
        if dy.is_cuda:
            return native.ext().maxpool_bwd(dy.contiguous(), idx, H, W)
        g = TF.max_unpool2d(dy.float().permute(0, 3, 1, 2), idx, 3, 2, 1, output_size=ctx.cpu_shape)
        return g.permute(0, 2, 3, 1).contiguous().to(dy.dtype)


def max_pool_3x3_s2(x):
    return MaxPool3x3s2Fn.apply(x)


class GlobalAvgPoolFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        N, H, W, C = x.shape
        ctx.shape = x.shape
        if x.is_cuda:
            return native.ext().avgpool(x.contiguous().view(N, H * W, C), H * W, False)
        return x.float().mean((1, 2)).to(x.dtype)

    @staticmethod
    def backward(ctx, dy):
        N, H, W, C = ctx.shape
        if dy.is_cuda:
            return native.ext().avgpool(dy.contiguous(), H * W, True).view(N, H, W, C)
        return (dy.float() / (H * W))[:, None, None, :].expand(N, H, W, C).contiguous().to(dy.dtype)


def global_avg_pool(x):
    return GlobalAvgPoolFn.apply(x)
