"""Convolution (im2col + GEMM), BatchNorm and pooling kernels against PyTorch fp32 on NCHW."""
import pytest
import torch
import torch.nn.functional as TF

from superscaler_b200.ops import conv as C
from superscaler_b200.ops import native

pytestmark = pytest.mark.gpu
DEV = "cuda"


def rel(a, b):
    a, b = a.float(), b.float()
    return ((a - b).abs().max() / (b.abs().max() + 1e-6)).item()


@pytest.mark.parametrize("cfg", [(2, 14, 14, 64, 128, 1, 1, 0), (2, 14, 14, 64, 128, 1, 2, 0), (2, 16, 16, 32, 64, 3, 1, 1),
                                 (2, 16, 16, 32, 64, 3, 2, 1), (2, 32, 32, 3, 32, 7, 2, 3), (1, 7, 7, 64, 64, 3, 1, 1)])
def test_conv2d_fwd_bwd(cfg):
    N, H, W, Cin, Cout, k, stride, pad = cfg
    torch.manual_seed(0)
    x = torch.randn(N, H, W, Cin, device=DEV).bfloat16()
    kpad = C._pad8(k * k * Cin)
    w = torch.zeros(Cout, kpad, device=DEV)
    w[:, :k * k * Cin] = torch.randn(Cout, k * k * Cin, device=DEV) * 0.1
    w = w.bfloat16()
    xr = x.float().requires_grad_(True)
    wr = w.float().requires_grad_(True)
    w4 = wr[:, :k * k * Cin].view(Cout, k, k, Cin).permute(0, 3, 1, 2)
    ref = TF.conv2d(xr.permute(0, 3, 1, 2), w4, stride=stride, padding=pad).permute(0, 2, 3, 1)
    dy = torch.randn_like(ref).bfloat16()
    ref.backward(dy.float())
    xg = x.clone().requires_grad_(Cin % 8 == 0)
    wg = w.clone().requires_grad_(True)
    y = C.conv2d(xg, wg, k, k, stride, pad)
    y.backward(dy)
    assert rel(y, ref) < 8e-3
    assert rel(wg.grad[:, :k * k * Cin], wr.grad[:, :k * k * Cin]) < 1.5e-2
    if Cin % 8 == 0:
        assert rel(xg.grad, xr.grad) < 1.5e-2
    torch.cuda.synchronize()
    assert native.check_status() == 0


@pytest.mark.parametrize("shape", [(4, 9, 9, 64), (3, 29, 31, 88), (16, 56, 56, 320)])
@pytest.mark.parametrize("relu,res", [(False, False), (True, False), (True, True)])
def test_batch_norm(relu, res, shape):
    """The middle shape has a column block that is only partly filled (88 channels = 11 groups of 8) and a row count
    that no block or unrolling factor divides; the last one has more rows than one pass of the grid covers."""
    torch.manual_seed(1)
    Cn = shape[-1]
    x = (torch.randn(*shape, device=DEV) * 2 + 1).bfloat16()
    r = torch.randn_like(x) if res else None
    g = (torch.rand(Cn, device=DEV) + 0.5).requires_grad_(True)
    b = torch.randn(Cn, device=DEV).requires_grad_(True)
    xr = x.float().requires_grad_(True)
    rr = r.float().requires_grad_(True) if res else None
    gr, br = g.detach().clone().requires_grad_(True), b.detach().clone().requires_grad_(True)
    ref = TF.batch_norm(xr.permute(0, 3, 1, 2), None, None, gr, br, True, 0.1, 1e-5).permute(0, 2, 3, 1)
    if res:
        ref = ref + rr
    if relu:
        ref = torch.relu(ref)
    dy = torch.randn_like(ref)
    ref.backward(dy)
    xg = x.clone().requires_grad_(True)
    rg = r.clone().requires_grad_(True) if res else None
    y = C.batch_norm(xg, g, b, rg, None, None, 1e-5, 0.1, relu)
    y.backward(dy.bfloat16())
    assert rel(y, ref) < 1e-2 and rel(xg.grad, xr.grad) < 3e-2
    assert rel(g.grad, gr.grad) < 2e-2 and rel(b.grad, br.grad) < 2e-2
    if res:
        assert rel(rg.grad, rr.grad) < 1e-2


@pytest.mark.parametrize("shape", [(2, 12, 12, 16), (3, 13, 11, 24), (2, 112, 112, 320)])
def test_pooling(shape):
    torch.manual_seed(2)
    x = torch.randn(*shape, device=DEV).bfloat16()
    xr = x.float().requires_grad_(True)
    ref = TF.max_pool2d(xr.permute(0, 3, 1, 2), 3, 2, 1).permute(0, 2, 3, 1)
    dy = torch.randn_like(ref)
    ref.backward(dy)
    xg = x.clone().requires_grad_(True)
    y = C.max_pool_3x3_s2(xg)
    y.backward(dy.bfloat16())
    assert rel(y, ref) < 1e-6 and rel(xg.grad, xr.grad) < 1e-2
    xa = x.clone().requires_grad_(True)
    ya = C.global_avg_pool(xa)
    ya.backward(torch.ones_like(ya))
    hw = shape[1] * shape[2]
    assert rel(ya, x.float().mean((1, 2))) < 8e-3 and rel(xa.grad, torch.full_like(x.float(), 1 / hw)) < 8e-3
