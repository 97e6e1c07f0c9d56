"""The kernels at the shapes the GPT-3 1.3B benchmark step runs them at (32768 rows = 16 sequences of 2048 tokens,
hidden 2048, 16 heads of 128, FFN 8192, vocabulary 51200), element by element against fp32 PyTorch.  Outputs too
large for a full fp32 restatement are compared on row blocks taken from the start, the middle and the ragged end."""
import math

import pytest
import torch

from superscaler_b200.ops import functional as F
from superscaler_b200.ops import native
from test_kernels_gpu import ATTN, ATTN_GRAD, close

pytestmark = pytest.mark.gpu
DEV = "cuda"
ROWS = 16 * 2048


@pytest.fixture(autouse=True)
def _status_clean():
    yield
    torch.cuda.synchronize()
    assert native.check_status() == 0, "a kernel's bounded wait ran out"


def _row_blocks(m, rows=512):
    return [slice(0, rows), slice(m // 2 - rows // 2 + 3, m // 2 + rows // 2 + 3), slice(m - rows, m)]


@pytest.mark.parametrize("shape", [(ROWS, 6144, 2048), (ROWS, 8192, 2048), (ROWS, 2048, 8192), (ROWS, 51200, 2048)])
def test_forward_gemm_with_bias_gelu_at_benchmark_shapes(shape):
    M, N, K = shape
    torch.manual_seed(41)
    A = torch.randn(M, K, device=DEV).bfloat16()
    B = (torch.randn(N, K, device=DEV) * 0.05).bfloat16()
    bias = torch.randn(N, device=DEV).bfloat16()
    pre = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    out = F.gemm(A, B, bias=bias, act=F.ACT_GELU, preact_out=pre)
    for rs in _row_blocks(M):
        v = A[rs].float() @ B.float().t() + bias.float()
        close(pre[rs], v, what=f"pre-activation {shape}")
        close(out[rs], F._gelu_tanh(v), what=f"bias gelu {shape}")


def test_dgrad_and_wgrad_at_benchmark_shapes():
    """dX = dY W (B stored MN-major) and dW += dY^T X (both MN-major, fp32 accumulation into the gradient buffer)."""
    M, N, K = ROWS, 2048, 8192          # the MLP down-projection: X [M, K], W [N, K], dY [M, N]
    torch.manual_seed(42)
    X = torch.randn(M, K, device=DEV).bfloat16()
    W = (torch.randn(N, K, device=DEV) * 0.05).bfloat16()
    dY = torch.randn(M, N, device=DEV).bfloat16()
    dX = F.gemm(dY, W, b_mn=True)
    for rs in _row_blocks(M):
        close(dX[rs], dY[rs].float() @ W.float(), what="dgrad")
    dW = torch.ones(N, K, device=DEV)
    F.gemm(dY, X, out=dW, a_mn=True, b_mn=True, accumulate=True)
    # 32768 products per element: the restatement runs in fp64 so that its own rounding stays out of the comparison,
    # and the tolerance allows the tensor core's fp32 accumulation over that depth (measured: 9e-5 of the rms)
    for rs in _row_blocks(N, 256):
        ref = (dY[:, rs].double().t() @ X.double() + 1).float()
        close(dW[rs], ref, what="wgrad fp32 accumulate", rtol=3e-4, atol_rms=3e-4)


def test_layernorm_at_benchmark_shape():
    H = 2048
    torch.manual_seed(43)
    x = torch.randn(ROWS, H, device=DEV).bfloat16()
    gam, bet = torch.randn(H, device=DEV), torch.randn(H, device=DEV)
    y, mean, rstd = native.ext().layernorm_fwd(x, None, gam, bet, 1e-5)
    close(y, torch.nn.functional.layer_norm(x.float(), (H,), gam, bet, 1e-5), what="layernorm fwd")
    dy = torch.randn_like(x)
    xr, gr, br = x.float().requires_grad_(True), gam.clone().requires_grad_(True), bet.clone().requires_grad_(True)
    torch.nn.functional.layer_norm(xr, (H,), gr, br, 1e-5).backward(dy.float())
    dg, db = torch.zeros(H, device=DEV), torch.zeros(H, device=DEV)
    dx = native.ext().layernorm_bwd(dy, x, gam, mean, rstd, None, dg, db, False)
    close(dx, xr.grad, what="layernorm dx")
    # 32768 addends per column: the fp32 partial sums differ in order from torch's
    close(dg, gr.grad, what="layernorm dgamma", rtol=1e-4, atol_rms=1e-4)
    close(db, br.grad, what="layernorm dbeta", rtol=1e-4, atol_rms=1e-4)


@pytest.mark.parametrize("deterministic", [False, True])
def test_flash_attention_at_benchmark_shape(deterministic):
    """16 heads of 128, 2048 tokens, causal (two sequences instead of sixteen: the fp32 restatement materialises the
    [batch, heads, S, S] scores); both backward forms -- the fused kernel and the dK/dV + dQ pair."""
    B, NH, S, HD = 2, 16, 2048, 128
    torch.manual_seed(44)
    h = NH * HD
    qkv = (torch.randn(B * S, 3 * h, device=DEV) * 0.5).bfloat16()
    do = torch.randn(B * S, h, device=DEV).bfloat16()
    qr = qkv.float().clone().requires_grad_(True)
    ref = F._attn_reference(qr[:, :h], qr[:, h:2 * h], qr[:, 2 * h:], B, NH, S, S, HD, 1.0 / math.sqrt(HD), True, None)
    ref.backward(do.float())
    was = native.ext().attn_bwd_deterministic()
    F.set_deterministic(deterministic)
    try:
        x = qkv.clone().requires_grad_(True)
        o = F.fused_qkv_attention(x, B, NH, S, HD, causal=True)
        o.backward(do)
    finally:
        F.set_deterministic(bool(was))
    # the absolute part of the tolerance is set by the first 256 queries: their elements have the size of single
    # terms, which is what the bf16 roundings inside the kernels are relative to; the rows behind them average
    # hundreds of terms and would pull a whole-tensor rms far below that
    close(o, ref, what="attention o", scale_of=ref[:256], **ATTN)
    for i, name in enumerate("qkv"):
        g_ref = qr.grad[:, i * h:(i + 1) * h]
        close(x.grad[:, i * h:(i + 1) * h], g_ref, what=f"attention d{name}", scale_of=g_ref[:256], **ATTN_GRAD)


def test_cross_entropy_at_benchmark_vocabulary():
    T, V = 4096, 51200
    torch.manual_seed(45)
    logits = (torch.randn(T, V, device=DEV) * 2).bfloat16()
    tg = torch.randint(0, V, (T,), device=DEV)
    lf = logits.float().clone().requires_grad_(True)
    ref = torch.nn.functional.cross_entropy(lf, tg, reduction="none")
    ref.sum().backward()
    st = native.ext().ce_stats(logits, tg, 0)
    loss = native.ext().ce_finalize(logits, tg, st, None, 0, 1.0, True)
    close(loss, ref, what="ce loss", rtol=1e-5, atol_rms=1e-5)
    close(logits, lf.grad, what="ce dlogits", rtol=8e-3, atol_rms=1e-4)


def test_adam_on_a_parameter_buffer_larger_than_l2():
    n = 64 * 1024 * 1024 + 5
    torch.manual_seed(46)
    p, g = torch.randn(n, device=DEV), torch.randn(n, device=DEV) * 1e-3
    m, v = torch.zeros(n, device=DEV), torch.zeros(n, device=DEV)
    p16 = torch.empty(n, device=DEV, dtype=torch.bfloat16)
    ss = torch.zeros(1, device=DEV)
    pr = p.clone().requires_grad_(True)
    opt = torch.optim.AdamW([pr], lr=1e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    pr.grad = g.clone()
    opt.step()
    native.ext().sumsq(g, ss, False)
    close(ss, (g.double() ** 2).sum()[None], what="sumsq", rtol=1e-5, atol_rms=0.0)
    native.ext().adam_step(p, m, v, g, p16, ss, None, 1e-3, 0.9, 0.95, 1e-8, 0.1, 1, 1.0, 1e9, n, True)
    close(p, pr.detach(), what="adam master", rtol=1e-6, atol_rms=1e-6)
    close(p16, pr.detach(), what="adam bf16 copy")
