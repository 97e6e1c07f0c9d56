"""Numerics of every sm_100a kernel against a plain PyTorch fp32 restatement of the same op."""
import math

import pytest
import torch

from superscaler_b200.ops import functional as F
from superscaler_b200.ops import native

pytestmark = pytest.mark.gpu
DEV = "cuda"


def rel(a, b):
    a, b = a.float(), b.float()
    return ((a - b).abs().max() / (b.abs().max() + 1e-6)).item()


def excess(a, ref, rtol, atol_rms, scale_of=None):
    """Largest |a - ref| / (atol_rms * rms(ref) + rtol * |ref|) over the elements: at most 1 when EVERY element is
    within its own tolerance, so an error in a small-magnitude element is not hidden by the tensor's largest value
    (which is all that `rel` looks at).  `scale_of`: the part of `ref` whose rms sets the absolute term (default: all)."""
    a, ref = a.float(), ref.float()
    tol = atol_rms * (ref if scale_of is None else scale_of.float()).pow(2).mean().sqrt() + rtol * ref.abs()
    return ((a - ref).abs() / tol).max().item()


def close(a, ref, rtol=8e-3, atol_rms=4e-3, what="", scale_of=None):
    """Per-element check; the defaults fit a bf16 result of fp32 arithmetic (half an ulp is 3.9e-3 relative)."""
    e = excess(a, ref, rtol, atol_rms, scale_of)
    print(f"[tol] {what or 'close'} rtol={rtol:g} atol_rms={atol_rms:g} excess={e:.3f}")
    assert e <= 1.0, f"{what}: element error {e:.2f} x its tolerance (rtol {rtol:g}, atol {atol_rms:g} x rms)"


FP32 = dict(rtol=2e-5, atol_rms=2e-5)         # fp32 results of fp32 accumulation
# Attention: P, dS and O (for delta = rowsum(dO * O)) pass through bf16 inside the kernels, and that rounding is
# relative to the TERMS of a row, not to its result.  In a causal row with one or two visible keys the terms are
# ten to thirty times the rms of the whole tensor (long rows average them down), so the absolute part of the
# tolerance has to be several per cent of that rms; measured worst elements: 2.5 % (O), 3.6 % (dQ), 2.1 % (dK).
ATTN = dict(rtol=1.6e-2, atol_rms=4e-2)
ATTN_GRAD = dict(rtol=2e-2, atol_rms=7e-2)


@pytest.fixture(autouse=True)
def _status_clean():
    yield
    torch.cuda.synchronize()
    assert native.check_status() == 0, "a kernel's bounded wait ran out"


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("shape", [(128, 128, 64), (256, 512, 256), (1000, 776, 520), (4096, 2048, 2048), (64, 96, 72)])
def test_gemm_variants(a_mn, b_mn, shape):
    M, N, K = shape
    torch.manual_seed(0)
    A = torch.randn(M, K, device=DEV).bfloat16()
    B = torch.randn(N, K, device=DEV).bfloat16()
    ref = A.float() @ B.float().t()
    a_in = A.t().contiguous() if a_mn else A
    b_in = B.t().contiguous() if b_mn else B
    out = F.gemm(a_in, b_in, a_mn=a_mn, b_mn=b_mn)
    assert rel(out, ref) < 6e-3
    close(out, ref, what="gemm bf16")
    acc = torch.ones(M, N, device=DEV)
    F.gemm(a_in, b_in, out=acc, a_mn=a_mn, b_mn=b_mn, accumulate=True)
    assert rel(acc, ref + 1) < 1e-4
    close(acc, ref + 1, what="gemm fp32 accumulate", **FP32)


@pytest.mark.parametrize("shape", [(640, 320, 50176), (1024, 1024, 16384), (96, 200, 4096)])
def test_weight_gradient_gemm_with_split_reduction(shape):
    """Small outputs with a long reduction are cut into K slices (one per otherwise idle SM) whose partial products
    are added in slice order: the result accumulates into an fp32 buffer like any other weight gradient and is the
    same on every run."""
    M, N, K = shape
    torch.manual_seed(17)
    assert native.ext().gemm_splitk_splits(M, N, K) > 1
    A = torch.randn(K, M, device=DEV).bfloat16()        # dY, MN-major
    B = torch.randn(K, N, device=DEV).bfloat16()        # X, MN-major
    ref = (A.double().t() @ B.double() + 1).float()
    outs = []
    for _ in range(2):
        acc = torch.ones(M, N, device=DEV)
        F.gemm(A, B, out=acc, a_mn=True, b_mn=True, accumulate=True)
        outs.append(acc)
    close(outs[0], ref, what="split-K wgrad", rtol=3e-4, atol_rms=3e-4)
    assert torch.equal(outs[0], outs[1])
    plain = torch.empty(M, N, device=DEV)
    F.gemm(A, B, out=plain, a_mn=True, b_mn=True)
    close(plain, ref - 1, what="split-K plain store", rtol=3e-4, atol_rms=3e-4)


def test_gemm_strided_operands():
    torch.manual_seed(1)
    big = torch.randn(300, 1024, device=DEV).bfloat16()
    A = big[:, 256:512]          # leading dimension 1024, 256 columns
    B = torch.randn(192, 256, device=DEV).bfloat16()
    out = torch.zeros(300, 384, device=DEV, dtype=torch.bfloat16)
    F.gemm(A, B, out=out[:, 64:256])
    assert rel(out[:, 64:256], A.float() @ B.float().t()) < 6e-3
    assert out[:, :64].abs().max() == 0 and out[:, 256:].abs().max() == 0


def test_gemm_epilogues():
    torch.manual_seed(2)
    M, N, K = 512, 768, 256
    A = torch.randn(M, K, device=DEV).bfloat16()
    B = (torch.randn(N, K, device=DEV) * 0.1).bfloat16()
    bias = torch.randn(N, device=DEV).bfloat16()
    res = torch.randn(M, N, device=DEV).bfloat16()
    pre = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    v = A.float() @ B.float().t() + bias.float()
    out = F.gemm(A, B, bias=bias, act=F.ACT_GELU, preact_out=pre, residual=res)
    assert rel(pre, v) < 6e-3
    close(pre, v, what="pre-activation")
    # the kernel applies GeLU to the fp32 value, the residual add rounds once more
    close(out, F._gelu_tanh(v) + res.float(), what="bias gelu residual")
    out = F.gemm(A, B, bias=bias, act=F.ACT_RELU)
    close(out, torch.relu(v), what="bias relu")
    aux = torch.randn(M, N, device=DEV).bfloat16()
    out = F.gemm(A, B, act=F.ACT_DGELU, aux=aux)
    close(out, (A.float() @ B.float().t()) * F._gelu_tanh_grad(aux.float()), what="dgelu")
    out = F.gemm(A, B, act=F.ACT_DRELU, aux=aux)
    close(out, (A.float() @ B.float().t()) * (aux.float() > 0), what="drelu")
    out = F.gemm(A, B, alpha=0.5, bias=bias.float())
    close(out, 0.5 * (A.float() @ B.float().t()) + bias.float(), what="alpha bias")


@pytest.mark.parametrize("epi", ["plain", "bias_gelu_preact", "dgelu", "drop_residual", "fp32_accumulate"])
def test_pair_gemm_epilogues_match_one_cta_kernel(epi):
    """The two-SM kernel (staged, coalesced epilogue) against the one-CTA kernel on a ragged shape that exercises
    full 64-column groups, a partly filled last N tile and a partly filled last M tile."""
    ext = native.ext()
    torch.manual_seed(31)
    M, N, K = 2500, 2112, 512
    A = torch.randn(M, K, device=DEV).bfloat16()
    B = (torch.randn(N, K, device=DEV) * 0.1).bfloat16()
    kw, outs = {}, ["out"]
    if epi == "bias_gelu_preact":
        kw = dict(bias=torch.randn(N, device=DEV).bfloat16(), act=F.ACT_GELU)
        outs.append("pre")
    elif epi == "dgelu":
        kw = dict(act=F.ACT_DGELU, aux=torch.randn(M, N, device=DEV).bfloat16())
    elif epi == "drop_residual":
        kw = dict(bias=torch.randn(N, device=DEV), dropout_p=0.1, seed=5, residual=torch.randn(M, N, device=DEV).bfloat16())
    res = {}
    try:
        for mode in (0, 1):
            ext.gemm_set_pair_mode(mode)
            if epi == "fp32_accumulate":
                out = torch.ones(M, N, device=DEV, dtype=torch.float32)
                F.gemm(A, B, out, accumulate=True)
            else:
                pre = torch.zeros(M, N, device=DEV, dtype=torch.bfloat16) if "pre" in outs else None
                out = F.gemm(A, B, preact_out=pre, **kw)
                if pre is not None:
                    res[("pre", mode)] = pre
            res[("out", mode)] = out
    finally:
        ext.gemm_set_pair_mode(1)
    torch.cuda.synchronize()
    assert native.check_status() == 0
    for name in outs:
        a, b = res[(name, 0)].float(), res[(name, 1)].float()
        # same math, but the compiler may contract multiply-adds differently in the two kernels
        assert (a - b).abs().max().item() <= 4e-3 * b.abs().max().item(), f"{epi}/{name}: {(a - b).abs().max().item()}"
    # and the two-SM kernel against fp32 arithmetic, every epilogue
    v = A.float() @ B.float().t()
    got = res[("out", 1)]
    if epi == "plain":
        close(got, v, what="pair plain")
    elif epi == "bias_gelu_preact":
        v = v + kw["bias"].float()
        close(res[("pre", 1)], v, what="pair pre-activation")
        close(got, F._gelu_tanh(v), what="pair bias gelu")
    elif epi == "dgelu":
        close(got, v * F._gelu_tanh_grad(kw["aux"].float()), what="pair dgelu")
    elif epi == "drop_residual":
        v = v + kw["bias"].float()
        r = kw["residual"].float()
        kept = got.float() != r                      # a dropped element is exactly the residual
        assert abs(kept.float().mean().item() - 230 / 256) < 5e-3
        full = v / (230 / 256) + r
        close(torch.where(kept, got.float(), full), full, what="pair dropout residual")
    else:
        close(got, v + 1, what="pair fp32 accumulate", **FP32)


def test_gemm_dropout_matches_elementwise_mask():
    torch.manual_seed(3)
    M, N, K = 256, 512, 128
    A = torch.randn(M, K, device=DEV).bfloat16()
    B = torch.randn(N, K, device=DEV).bfloat16()
    v = A.float() @ B.float().t()
    out = F.gemm(A, B, dropout_p=0.1, seed=77)
    kept = out != 0
    frac = kept.float().mean().item()
    assert abs(frac - 0.9) < 0.01
    assert rel(out[kept], (v / (230 / 256))[kept]) < 6e-3   # keep probability quantised to 1/256
    ones = torch.ones(M, N, device=DEV, dtype=torch.bfloat16)
    m_fwd = native.ext().elementwise(F.EW_DROPOUT, ones, None, None, 0.1, 77) != 0
    m_bwd = native.ext().elementwise(F.EW_DROPOUT_BWD, ones, None, None, 0.1, 77) != 0
    assert bool((m_fwd == kept).all()) and bool((m_bwd == kept).all())
    other = native.ext().elementwise(F.EW_DROPOUT, ones, None, None, 0.1, 78) != 0
    assert not bool((other == kept).all())


@pytest.mark.parametrize("H", [512, 1024, 2048, 4096, 1536])
def test_layernorm(H):
    torch.manual_seed(4)
    x = torch.randn(777, H, device=DEV).bfloat16()
    gam, bet = torch.randn(H, device=DEV), torch.randn(H, device=DEV)
    y, mean, rstd = native.ext().layernorm_fwd(x, None, gam, bet, 1e-5)
    ref = torch.nn.functional.layer_norm(x.float(), (H,), gam, bet, 1e-5)
    assert rel(y, ref) < 6e-3
    close(y, ref, what="layernorm fwd")
    dy = torch.randn_like(x)
    xr, gr, br = x.float().requires_grad_(True), gam.clone().requires_grad_(True), bet.clone().requires_grad_(True)
    torch.nn.functional.layer_norm(xr, (H,), gr, br, 1e-5).backward(dy.float())
    dg, db = torch.zeros(H, device=DEV), torch.zeros(H, device=DEV)
    dx = native.ext().layernorm_bwd(dy, x, gam, mean, rstd, None, dg, db, False)
    assert rel(dx, xr.grad) < 6e-3 and rel(dg, gr.grad) < 1e-4 and rel(db, br.grad) < 1e-4
    close(dx, xr.grad, what="layernorm dx")
    close(dg, gr.grad, what="layernorm dgamma", rtol=1e-4, atol_rms=1e-4)
    close(db, br.grad, what="layernorm dbeta", rtol=1e-4, atol_rms=1e-4)
    native.ext().layernorm_bwd(dy, x, gam, mean, rstd, None, dg, db, True)
    assert rel(dg, 2 * gr.grad) < 1e-4


def test_layernorm_residual_prologue():
    torch.manual_seed(5)
    H = 2048
    x, r = torch.randn(100, H, device=DEV).bfloat16(), torch.randn(100, H, device=DEV).bfloat16()
    gam, bet = torch.ones(H, device=DEV), torch.zeros(H, device=DEV)
    y, mean, rstd, s = native.ext().layernorm_fwd(x, r, gam, bet, 1e-5)
    sref = (x.float() + r.float()).bfloat16()
    assert torch.equal(s, sref)
    assert rel(y, torch.nn.functional.layer_norm(sref.float(), (H,), gam, bet, 1e-5)) < 6e-3


def test_colsum_and_elementwise():
    torch.manual_seed(6)
    a = torch.randn(1000, 512, device=DEV).bfloat16()
    out = torch.zeros(512, device=DEV)
    native.ext().colsum(a, out, False)
    assert rel(out, a.float().sum(0)) < 1e-5
    x = torch.randn(300, 1024, device=DEV).bfloat16()
    b = torch.randn(1024, device=DEV).bfloat16()
    r, g = torch.randn_like(x), torch.randn_like(x)
    e = native.ext().elementwise
    assert rel(e(F.EW_BIAS_GELU, x, None, b, 0.0, 0), F._gelu_tanh(x.float() + b.float())) < 6e-3
    assert rel(e(F.EW_BIAS_GELU_BWD, x, g, b, 0.0, 0), g.float() * F._gelu_tanh_grad(x.float() + b.float())) < 6e-3
    assert rel(e(F.EW_BIAS_DROP_ADD, x, r, b, 0.0, 0), x.float() + b.float() + r.float()) < 6e-3
    assert rel(e(F.EW_RELU, x, None, b, 0.0, 0), torch.relu(x.float() + b.float())) < 6e-3
    assert rel(e(F.EW_RELU_BWD, x, g, b, 0.0, 0), g.float() * ((x.float() + b.float()) > 0)) < 6e-3
    assert rel(e(F.EW_ADD, x, r, None, 0.0, 0), x.float() + r.float()) < 6e-3
    keep = (e(F.EW_DROPOUT, x, None, None, 0.25, 5) != 0).float().mean().item()
    assert abs(keep - 0.75) < 0.01


def test_softmax_family():
    torch.manual_seed(7)
    x = torch.randn(2, 4, 256, 256, device=DEV).bfloat16()
    tri = torch.ones(256, 256, dtype=torch.bool, device=DEV).tril()
    y = F.scaled_softmax(x, 0.5, 1)
    ref = torch.softmax((x.float() * 0.5).masked_fill(~tri, float("-inf")), -1)
    assert rel(y, ref) < 6e-3
    g = torch.randn_like(x)
    dx = native.ext().softmax_bwd(g, y, 0.5)
    yf = y.float()
    assert rel(dx, 0.5 * (g.float() * yf - yf * (g.float() * yf).sum(-1, keepdim=True))) < 6e-3
    mask = (torch.rand(2, 1, 256, 256, device=DEV) < 0.2).to(torch.uint8)
    y = F.scaled_softmax(x, 0.5, 2, mask)
    assert rel(y, torch.softmax((x.float() * 0.5).masked_fill(mask.bool(), -10000.0), -1)) < 6e-3
    y = F.scaled_softmax(x, 0.5, 0)
    assert rel(y, torch.softmax(x.float() * 0.5, -1)) < 6e-3


def test_adam_and_sumsq():
    torch.manual_seed(8)
    n = 1_000_003
    p, g = torch.randn(n, device=DEV), torch.randn(n, device=DEV)
    m, v = torch.zeros(n, device=DEV), torch.zeros(n, device=DEV)
    p16 = torch.empty(n, device=DEV, dtype=torch.bfloat16)
    ss = torch.zeros(1, device=DEV)
    native.ext().sumsq(g, ss, False)
    assert rel(ss, (g.double() ** 2).sum()[None]) < 1e-5
    pr = p.clone().requires_grad_(True)
    opt = torch.optim.AdamW([pr], lr=1e-2, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01)
    for step in (1, 2):
        gg = torch.randn(n, device=DEV)
        g.copy_(gg)
        native.ext().sumsq(g, ss, False)
        clip = min(1.0, 1.0 / (gg.norm().item() + 1e-6))
        pr.grad = gg * clip
        opt.step()
        native.ext().adam_step(p, m, v, g, p16, ss, None, 1e-2, 0.9, 0.999, 1e-8, 0.01, step, 1.0, 1.0, n, True)
    assert rel(p, pr.detach()) < 1e-5 and rel(p16, pr.detach()) < 6e-3 and float(g.abs().max()) == 0.0
    # non-finite gradients: the step is skipped on the device and reported
    skipped = torch.zeros(1, device=DEV, dtype=torch.int32)
    before = p.clone()
    ss.fill_(float("inf"))
    native.ext().adam_step(p, m, v, g, p16, ss, skipped, 1e-2, 0.9, 0.999, 1e-8, 0.01, 3, 1.0, 1.0, n, True)
    assert torch.equal(p, before) and int(skipped.item()) == 1


def test_embedding_and_cross_entropy():
    torch.manual_seed(9)
    V, H, T = 1000, 512, 300
    W, P = torch.randn(V, H, device=DEV).bfloat16(), torch.randn(64, H, device=DEV).bfloat16()
    ids, pos = torch.randint(0, V, (T,), device=DEV), torch.randint(0, 64, (T,), device=DEV)
    out = native.ext().embedding_fwd(ids, pos, W, P, 0, 0.0, 0)
    assert rel(out, W.float()[ids] + P.float()[pos]) < 6e-3
    half = native.ext().embedding_fwd(ids, None, W[500:].contiguous(), None, 500, 0.0, 0)
    refh = torch.where((ids >= 500)[:, None], W.float()[ids], torch.zeros(1, device=DEV))
    assert rel(half, refh) < 6e-3
    g = torch.randn(T, H, device=DEV).bfloat16()
    dW, dP = torch.zeros(V, H, device=DEV), torch.zeros(64, H, device=DEV)
    native.ext().embedding_bwd(ids, pos, g, dW, dP, 0, 0.0, 0)
    assert rel(dW, torch.zeros(V, H, device=DEV).index_add_(0, ids, g.float())) < 1e-5
    assert rel(dP, torch.zeros(64, H, device=DEV).index_add_(0, pos, g.float())) < 1e-5
    Vv = 5000
    logits = (torch.randn(T, Vv, device=DEV) * 3).bfloat16()
    tg = torch.randint(0, Vv, (T,), device=DEV)
    lf = logits.float().clone().requires_grad_(True)
    ref = torch.nn.functional.cross_entropy(lf, tg, reduction="none")
    ref.sum().backward()
    st = native.ext().ce_stats(logits, tg, 0)
    loss = native.ext().ce_finalize(logits, tg, st, None, 0, 1.0, True)
    assert rel(loss, ref) < 1e-4 and rel(logits, lf.grad) < 6e-3
    close(loss, ref, what="ce loss", rtol=1e-5, atol_rms=1e-5)
    close(logits, lf.grad, what="ce dlogits", rtol=8e-3, atol_rms=1e-4)


def test_sorted_embedding_backward_is_exact_and_repeatable():
    """The run-by-run scatter equals the fp32 index_add, also with dropout (against the atomic kernel, which draws
    the same mask), for a vocabulary shard, and gives bitwise equal results when repeated."""
    torch.manual_seed(12)
    V, H, T = 700, 2048, 4096
    ids = torch.randint(0, V, (T,), device=DEV)
    ids[::7] = 3                                    # one heavily repeated token
    pos = torch.arange(T, device=DEV) % 128
    g = torch.randn(T, H, device=DEV).bfloat16()

    def sorted_grad(keys_t, rows, k0, p, seed):
        out = torch.zeros(rows, H, device=DEV)
        keys, order = torch.sort(keys_t, stable=True)
        native.ext().embedding_bwd_sorted(keys, order, g, out, k0, p, seed)
        return out

    dW = sorted_grad(ids, V, 0, 0.0, 0)
    assert rel(dW, torch.zeros(V, H, device=DEV).index_add_(0, ids, g.float())) < 1e-6
    dP = sorted_grad(pos, 128, 0, 0.0, 0)
    assert rel(dP, torch.zeros(128, H, device=DEV).index_add_(0, pos, g.float())) < 1e-6
    shard = sorted_grad(ids, 300, 400, 0.0, 0)      # rows 400..699 only
    assert rel(shard, torch.zeros(V, H, device=DEV).index_add_(0, ids, g.float())[400:]) < 1e-6
    aW, aP = torch.zeros(V, H, device=DEV), torch.zeros(128, H, device=DEV)
    native.ext().embedding_bwd(ids, pos, g, aW, aP, 0, 0.1, 77)
    assert rel(sorted_grad(ids, V, 0, 0.1, 77), aW) < 1e-5 and rel(sorted_grad(pos, 128, 0, 0.1, 77), aP) < 1e-5
    assert torch.equal(sorted_grad(ids, V, 0, 0.1, 77), sorted_grad(ids, V, 0, 0.1, 77))
    assert native.check_status() == 0


@pytest.mark.parametrize("cfg", [(1, 1, 128, 128, False), (1, 2, 256, 128, True), (2, 3, 512, 128, True),
                                 (2, 2, 256, 64, True), (1, 2, 384, 64, False), (1, 2, 200, 128, False)])
def test_flash_attention_fwd_bwd(cfg):
    B, NH, S, HD, causal = cfg
    torch.manual_seed(10)
    h = NH * HD
    qkv = (torch.randn(B * S, 3 * h, device=DEV) * 0.5).bfloat16()
    scale = 1.0 / math.sqrt(HD)
    qr = qkv.float().clone().requires_grad_(True)
    ref = F._attn_reference(qr[:, :h], qr[:, h:2 * h], qr[:, 2 * h:], B, NH, S, S, HD, scale, causal, None)
    do = torch.randn(B * S, h, device=DEV).bfloat16()
    ref.backward(do.float())
    x = qkv.clone().requires_grad_(True)
    o = F.fused_qkv_attention(x, B, NH, S, HD, causal=causal)
    o.backward(do)
    assert rel(o, ref) < 8e-3
    close(o, ref, what="attention o", **ATTN)
    for lo in (0, h, 2 * h):
        assert rel(x.grad[:, lo:lo + h], qr.grad[:, lo:lo + h]) < 1.5e-2
        close(x.grad[:, lo:lo + h], qr.grad[:, lo:lo + h], what=f"attention grad {lo // h}", **ATTN_GRAD)


def test_flash_attention_cross_and_kv_lens():
    torch.manual_seed(11)
    B, NH, SQ, SK, HD = 2, 2, 128, 384, 64
    h = NH * HD
    q = (torch.randn(B * SQ, h, device=DEV) * 0.5).bfloat16().requires_grad_(True)
    kv = (torch.randn(B * SK, 2 * h, device=DEV) * 0.5).bfloat16().requires_grad_(True)
    lens = torch.tensor([384, 250], device=DEV, dtype=torch.int32)
    scale = 1.0 / math.sqrt(HD)
    o = F.flash_attention(q, kv, kv, B, NH, SQ, SK, HD, cols=(0, 0, h), scale=scale, kv_lens=lens)
    do = torch.randn_like(o)
    o.backward(do)
    qr, kvr = q.detach().float().requires_grad_(True), kv.detach().float().requires_grad_(True)
    ref = F._attn_reference(qr, kvr[:, :h], kvr[:, h:], B, NH, SQ, SK, HD, scale, False, lens)
    ref.backward(do.float())
    assert rel(o, ref) < 8e-3 and rel(q.grad, qr.grad) < 1.5e-2 and rel(kv.grad, kvr.grad) < 1.5e-2


def test_flash_attention_dropout_consistency():
    """With dropout the three kernels must regenerate one mask: check dV = P_drop^T dO through linearity in V."""
    torch.manual_seed(12)
    B, NH, S, HD = 1, 2, 256, 128
    h = NH * HD
    qkv = (torch.randn(B * S, 3 * h, device=DEV) * 0.5).bfloat16()
    x = qkv.clone().requires_grad_(True)
    o = F.fused_qkv_attention(x, B, NH, S, HD, causal=True, dropout_p=0.2, seed=99)
    o2 = F.fused_qkv_attention(qkv, B, NH, S, HD, causal=True, dropout_p=0.2, seed=99)
    assert torch.equal(o, o2)
    do = torch.randn_like(o)
    o.backward(do)
    # O is linear in V for a fixed mask: <dO, O(V)> = <dV, V>
    lhs = (do.float() * o.float()).sum()
    rhs = (x.grad[:, 2 * h:].float() * qkv[:, 2 * h:].float()).sum()
    assert abs(lhs - rhs) / (abs(lhs) + 1e-6) < 2e-2
    o_nodrop = F.fused_qkv_attention(qkv, B, NH, S, HD, causal=True)
    assert rel(o, o_nodrop) > 0.05  # dropout really changes the output


def test_flash_attention_dropout_grads_with_extracted_mask():
    """Reads the dropout mask out of the forward kernel (V = one-hot blocks gives P_drop itself), then checks dQ, dK,
    dV of the backward kernels against autograd through plain fp32 attention that uses that mask."""
    torch.manual_seed(21)
    B, NH, S, HD, pdrop, seed = 1, 2, 256, 128, 0.25, 5
    h = NH * HD
    qkv = (torch.randn(B * S, 3 * h, device=DEV) * 0.5).bfloat16()
    pd = torch.zeros(NH, S, S, device=DEV)
    eye = torch.eye(HD, device=DEV)
    for blk in range(S // HD):
        v = torch.zeros(S, NH, HD, device=DEV)
        v[blk * HD:(blk + 1) * HD] = eye[:, None, :]
        x = qkv.clone()
        x[:, 2 * h:] = v.reshape(S, h).bfloat16()
        o = F.fused_qkv_attention(x, B, NH, S, HD, causal=True, dropout_p=pdrop, seed=seed)
        pd[:, :, blk * HD:(blk + 1) * HD] = o.float().view(S, NH, HD).permute(1, 0, 2)
    mask = (pd != 0).float()
    causal = torch.tril(torch.ones(S, S, device=DEV))
    kept = (mask * causal).sum() / causal.sum() / NH
    assert abs(kept.item() - 0.75) < 0.02, kept          # 192 / 256 of the visible entries survive
    x = qkv.clone().requires_grad_(True)
    o = F.fused_qkv_attention(x, B, NH, S, HD, causal=True, dropout_p=pdrop, seed=seed)
    do = torch.randn_like(o)
    o.backward(do)
    xr = qkv.float().clone().requires_grad_(True)
    q, k, v = (xr[:, i * h:(i + 1) * h].view(S, NH, HD).permute(1, 0, 2) for i in range(3))
    sc = (q @ k.transpose(1, 2)) * HD ** -0.5
    sc = sc.masked_fill(causal == 0, float("-inf"))
    pr = torch.softmax(sc, -1) * mask * (256.0 / 192.0)
    ref = (pr @ v).permute(1, 0, 2).reshape(S, h)
    ref.backward(do.float())
    assert rel(o, ref) < 1e-2
    for i, name in enumerate("qkv"):
        assert rel(x.grad[:, i * h:(i + 1) * h], xr.grad[:, i * h:(i + 1) * h]) < 2e-2, name


def test_lm_head_cross_entropy_autograd():
    torch.manual_seed(13)
    T, H, V = 256, 256, 1024
    x = torch.randn(T, H, device=DEV).bfloat16().requires_grad_(True)
    W = (torch.randn(V, H, device=DEV) * 0.05).bfloat16().requires_grad_(True)
    tg = torch.randint(0, V, (T,), device=DEV)
    loss = F.lm_head_cross_entropy(x, W, tg, None, 0, 1.0 / T)
    loss.backward()
    xr, wr = x.detach().float().requires_grad_(True), W.detach().float().requires_grad_(True)
    ref = torch.nn.functional.cross_entropy(xr @ wr.t(), tg)
    ref.backward()
    assert abs(loss.item() - ref.item()) < 2e-2
    assert rel(x.grad, xr.grad) < 3e-2 and rel(W.grad, wr.grad) < 3e-2


def test_peer_wait_times_out_with_status_when_signal_is_withheld():
    """A collective kernel whose peer never posts its flag must return within its time limit and report
    kStatusPeerTimeout; the context stays usable.  The 'peer' is a second set of local buffers that nothing writes."""
    import time
    ext = native.ext()
    n = 1 << 16
    bufs = [torch.zeros(n, device=DEV), torch.zeros(n, device=DEV)]
    flags = [torch.zeros(ext.comm_max_blocks() * 2, device=DEV, dtype=torch.int32) for _ in range(2)]
    peer_ptrs = torch.tensor([b.data_ptr() for b in bufs], dtype=torch.int64, device=DEV)
    flag_ptrs = torch.tensor([f.data_ptr() for f in flags], dtype=torch.int64, device=DEV)
    torch.cuda.synchronize()
    assert native.check_status() == 0
    ext.comm_set_peer_timeout_ms(200.0)
    try:
        t0 = time.time()
        ext.allreduce_scale_f32(peer_ptrs, 0, flag_ptrs, 0, 2, n, 1.0, 1)     # rank 0 of 2; rank 1 never arrives
        torch.cuda.synchronize()
        assert time.time() - t0 < 10.0
        assert int(ext.status().item()) == 2                                   # kStatusPeerTimeout
    finally:
        ext.comm_set_peer_timeout_ms(0.0)                                      # back to the default
        ext.status().zero_()
    # the context is intact: a normal kernel still runs
    a = torch.randn(256, 128, device=DEV).bfloat16()
    assert torch.isfinite(F.gemm(a, a).float()).all()
    assert native.check_status() == 0


@pytest.mark.parametrize("cfg", [(2, 4, 256, 64, False, 0.0), (1, 2, 384, 64, True, 0.0), (2, 2, 256, 128, False, 0.0)])
def test_flash_attention_relative_position_bias(cfg):
    """Scores with a per-head bias that depends on key - query (T5 relative-position buckets): forward, dQ / dK / dV and
    the gradient of the distance table against plain fp32 attention with the materialised [heads, S, S] bias."""
    from superscaler_b200.models.relative_position import bias_from_table
    B, NH, S, HD, causal, _ = cfg
    torch.manual_seed(31)
    h = NH * HD
    qkv = (torch.randn(B * S, 3 * h, device=DEV) * 0.5).bfloat16()
    table = (torch.randn(NH, 2 * S - 1, device=DEV) * 0.5)
    lens = None if causal else torch.tensor([S, S - 37][:B] + [S] * (B - 2), device=DEV, dtype=torch.int32)
    scale = 1.0 / math.sqrt(HD)
    do = torch.randn(B * S, h, device=DEV).bfloat16()
    x = qkv.clone().requires_grad_(True)
    t = table.clone().requires_grad_(True)
    o = F.flash_attention(x, x, x, B, NH, S, S, HD, cols=(0, h, 2 * h), scale=scale, causal=causal, kv_lens=lens,
                          bias_table=t)
    o.backward(do)
    xr = qkv.float().clone().requires_grad_(True)
    tr = table.clone().requires_grad_(True)
    ref = F.attention_with_bias(xr, B, NH, S, HD, scale, causal, lens, bias_from_table(tr, S, S))
    ref.backward(do.float())
    assert rel(o, ref) < 1e-2
    for lo in (0, h, 2 * h):
        assert rel(x.grad[:, lo:lo + h], xr.grad[:, lo:lo + h]) < 2e-2
    assert rel(t.grad, tr.grad) < 2e-2
    assert native.check_status() == 0
