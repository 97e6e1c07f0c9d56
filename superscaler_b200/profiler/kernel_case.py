"""Runs ONE kernel family on a small, fixed case: the command to put under a kernel profiler, and a quick timing
check.  Inputs exceed the L2 cache so that memory counters stay meaningful, but stay far below a GB.

    python -m superscaler_b200.profiler.kernel_case gemm 16384 8192 2048 [--a-mn] [--b-mn] [--single]
    python -m superscaler_b200.profiler.kernel_case attention 2 16 2048 128 [--dropout 0.1]
    python -m superscaler_b200.profiler.kernel_case layernorm 32768 2048
    python -m superscaler_b200.profiler.kernel_case embedding 32768 2048 51200 [--dropout 0.1]
    python -m superscaler_b200.profiler.kernel_case crossentropy 4096 51200
    python -m superscaler_b200.profiler.kernel_case adam 100000000
    python -m superscaler_b200.profiler.kernel_case colsum 32768 8192
    python -m superscaler_b200.profiler.kernel_case convbn 32 56 640 [--filter 3]

Prints one line per kernel family: milliseconds per call (CUDA events, after warm-up) and TFLOP/s.
"""
from __future__ import annotations

import argparse

import torch

from ..ops import functional as F
from ..ops import native


def _time(fn, warmup: int, iters: int) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def run_gemm(a) -> None:
    ext = native.ext()
    ext.gemm_set_pair_mode(0 if a.single else 1)
    torch.manual_seed(0)
    A = torch.randn((a.K, a.M) if a.a_mn else (a.M, a.K), device="cuda").bfloat16()
    B = torch.randn((a.K, a.N) if a.b_mn else (a.N, a.K), device="cuda").bfloat16()
    out = torch.empty(a.M, a.N, device="cuda", dtype=torch.bfloat16)
    kw = {}
    if a.epilogue == "gelu":      # bias + pre-activation store + GeLU (MLP up-projection forward)
        kw = dict(bias=torch.zeros(a.N, device="cuda", dtype=torch.bfloat16), act=F.ACT_GELU,
                  preact_out=torch.empty_like(out))
    elif a.epilogue == "dgelu":   # GeLU derivative from the saved pre-activation (MLP down-projection dgrad)
        kw = dict(act=F.ACT_DGELU, aux=torch.randn(a.M, a.N, device="cuda").bfloat16())
    elif a.epilogue == "dropadd":  # bias + dropout + residual (attention output / MLP down-projection forward)
        kw = dict(bias=torch.zeros(a.N, device="cuda", dtype=torch.bfloat16), dropout_p=0.1, seed=7,
                  residual=torch.randn(a.M, a.N, device="cuda").bfloat16())
    ms = _time(lambda: F.gemm(A, B, out, a_mn=a.a_mn, b_mn=a.b_mn, **kw), a.warmup, a.iters)
    print(f"gemm {a.M}x{a.N}x{a.K} a_mn={a.a_mn} b_mn={a.b_mn} pair={not a.single} epilogue={a.epilogue}: {ms:.4f} ms "
          f"{2 * a.M * a.N * a.K / ms / 1e9:.0f} TFLOP/s status {int(ext.status().item())}")


def run_attention(a) -> None:
    ext = native.ext()
    B_, NH, S, HD = a.B, a.NH, a.S, a.HD
    h = NH * HD
    torch.manual_seed(0)
    qkv = (torch.randn(B_ * S, 3 * h, device="cuda") * 0.5).bfloat16()
    sc = HD ** -0.5
    fwd = lambda: ext.attn_fwd(qkv, qkv, qkv, B_, NH, S, S, HD, 0, h, 2 * h, sc, True, None, a.dropout, 1234, None)
    o, lse = fwd()
    do = torch.randn_like(o)
    dqkv = torch.empty_like(qkv)
    bwd = lambda: ext.attn_bwd(qkv, qkv, qkv, o, lse, do, dqkv, dqkv, dqkv, B_, NH, S, S, HD, 0, h, 2 * h, 0, h, 2 * h,
                               sc, True, None, a.dropout, 1234, None, None)
    ext.set_attn_bwd_deterministic(bool(a.pair))     # --pair: the dK/dV + dQ kernel pair instead of the fused kernel
    flops = 4 * B_ * NH * S * S * HD * 0.5    # causal
    for name, fn, mult in (("fwd", fwd, 1.0), ("bwd", bwd, 2.5)):
        ms = _time(fn, a.warmup, a.iters)
        print(f"attention {name} B{B_} NH{NH} S{S} HD{HD} causal dropout={a.dropout}: {ms:.4f} ms "
              f"{flops * mult / ms / 1e9:.0f} TFLOP/s status {int(ext.status().item())}")


def run_layernorm(a) -> None:
    """LayerNorm forward and backward (dx, and the gamma / beta gradients accumulated into fp32 buffers)."""
    ext = native.ext()
    torch.manual_seed(0)
    x = torch.randn(a.rows, a.H, device="cuda").bfloat16()
    dy = torch.randn_like(x)
    gamma, beta = torch.ones(a.H, device="cuda"), torch.zeros(a.H, device="cuda")
    dg, db = torch.zeros_like(gamma), torch.zeros_like(beta)
    y, mean, rstd = ext.layernorm_fwd(x, None, gamma, beta, 1e-5)
    nbytes = x.numel() * 2
    for name, fn, moved in (("fwd", lambda: ext.layernorm_fwd(x, None, gamma, beta, 1e-5), 2 * nbytes),
                            ("bwd", lambda: ext.layernorm_bwd(dy, x, gamma, mean, rstd, None, dg, db, True),
                             3 * nbytes)):
        ms = _time(fn, a.warmup, a.iters)
        print(f"layernorm {name} {a.rows}x{a.H}: {ms:.4f} ms {moved / ms / 1e6:.0f} GB/s (algorithmic bytes) "
              f"status {int(ext.status().item())}")


def run_embedding(a) -> None:
    """Embedding forward (word + position + dropout) and the two forms of its backward scatter."""
    ext = native.ext()
    torch.manual_seed(0)
    T, H, V = a.tokens, a.H, a.V
    seq = min(2048, T)
    ids = torch.randint(0, V, (T,), device="cuda")
    pos = torch.arange(T, device="cuda") % seq
    W = torch.randn(V, H, device="cuda").bfloat16()
    P = torch.randn(seq, H, device="cuda").bfloat16()
    g = torch.randn(T, H, device="cuda").bfloat16()
    dW, dP = torch.zeros(V, H, device="cuda"), torch.zeros(seq, H, device="cuda")

    def sorted_bwd():
        for keys_t, dst in ((ids, dW), (pos, dP)):
            keys, order = torch.sort(keys_t, stable=True)
            ext.embedding_bwd_sorted(keys, order, g, dst, 0, a.dropout, 5)

    cases = (("fwd", lambda: ext.embedding_fwd(ids, pos, W, P, 0, a.dropout, 5), 3 * T * H * 2),
             ("bwd sorted runs", sorted_bwd, T * H * 2 + 2 * T * H * 4),
             ("bwd float atomics", lambda: ext.embedding_bwd(ids, pos, g, dW, dP, 0, a.dropout, 5),
              T * H * 2 + 2 * T * H * 4))
    for name, fn, moved in cases:
        ms = _time(fn, a.warmup, a.iters)
        print(f"embedding {name} tokens {T} H {H} V {V} dropout={a.dropout}: {ms:.4f} ms "
              f"{moved / ms / 1e6:.0f} GB/s (algorithmic bytes) status {int(ext.status().item())}")


def run_crossentropy(a) -> None:
    """Row statistics of bf16 logits, then loss + in-place gradient (the two passes of the LM-head loss)."""
    ext = native.ext()
    torch.manual_seed(0)
    logits = (torch.randn(a.tokens, a.V, device="cuda") * 2).bfloat16()
    tg = torch.randint(0, a.V, (a.tokens,), device="cuda")
    st = ext.ce_stats(logits, tg, 0)
    nbytes = logits.numel() * 2
    for name, fn, moved in (("stats", lambda: ext.ce_stats(logits, tg, 0), nbytes),
                            ("finalize", lambda: ext.ce_finalize(logits, tg, st, None, 0, 1.0, True), 2 * nbytes)):
        ms = _time(fn, a.warmup, a.iters)
        print(f"cross-entropy {name} tokens {a.tokens} V {a.V}: {ms:.4f} ms {moved / ms / 1e6:.0f} GB/s "
              f"(algorithmic bytes) status {int(ext.status().item())}")


def run_colsum(a) -> None:
    """Column sums of a bf16 matrix (bias gradients)."""
    ext = native.ext()
    torch.manual_seed(0)
    x = torch.randn(a.rows, a.N, device="cuda").bfloat16()
    out = torch.zeros(a.N, device="cuda")
    ms = _time(lambda: ext.colsum(x, out, True), a.warmup, a.iters)
    print(f"colsum {a.rows}x{a.N}: {ms:.4f} ms {x.numel() * 2 / ms / 1e6:.0f} GB/s (algorithmic bytes) "
          f"status {int(ext.status().item())}")


def run_adam(a) -> None:
    """Squared gradient norm, then the fused Adam step (fp32 master, moments, gradient zeroing, bf16 copy)."""
    ext = native.ext()
    torch.manual_seed(0)
    n = a.n
    p, g = torch.randn(n, device="cuda"), torch.randn(n, device="cuda") * 1e-3
    m, v = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    p16 = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    ss = torch.zeros(1, device="cuda")
    step = lambda: ext.adam_step(p, m, v, g, p16, ss, None, 1e-4, 0.9, 0.95, 1e-8, 0.1, 1, 1.0, 1.0, n, True)
    for name, fn, moved in (("sumsq", lambda: ext.sumsq(g, ss, False), 4 * n), ("adam", step, (4 * 4 + 3 * 4 + 2) * n)):
        ms = _time(fn, a.warmup, a.iters)
        print(f"optimizer {name} n {n}: {ms:.4f} ms {moved / ms / 1e6:.0f} GB/s (algorithmic bytes) "
              f"status {int(ext.status().item())}")


def run_convbn(a) -> None:
    """One Wide-ResNet bottleneck-sized k x k convolution (patch matrix + GEMM; dgrad + scatter back) and the
    BatchNorm + ReLU around it, NHWC bf16."""
    from ..ops import conv as C
    ext = native.ext()
    torch.manual_seed(0)
    N, HW, Cn, k = a.N, a.HW, a.C, a.filter
    x = torch.randn(N, HW, HW, Cn, device="cuda").bfloat16().requires_grad_(True)
    w = (torch.randn(Cn, C._pad8(k * k * Cn), device="cuda") * 0.02).bfloat16().requires_grad_(True)
    gamma, beta = torch.ones(Cn, device="cuda", requires_grad=True), torch.zeros(Cn, device="cuda", requires_grad=True)
    rm, rv = torch.zeros(Cn, device="cuda"), torch.ones(Cn, device="cuda")

    def fwd_bwd():
        y = C.batch_norm(C.conv2d(x, w, k, k, 1, k // 2), gamma, beta, None, rm, rv, relu=True)
        y.backward(y.detach())
        x.grad = w.grad = gamma.grad = beta.grad = None

    ms = _time(fwd_bwd, a.warmup, a.iters)
    flops = 3 * 2 * N * HW * HW * Cn * Cn * k * k
    print(f"conv{k}x{k} + batch-norm + relu, forward and backward, N{N} {HW}x{HW}x{Cn}: {ms:.4f} ms "
          f"{flops / ms / 1e9:.0f} TFLOP/s status {int(ext.status().item())}")


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="kind", required=True)
    g = sub.add_parser("gemm")
    g.add_argument("M", type=int), g.add_argument("N", type=int), g.add_argument("K", type=int)
    g.add_argument("--a-mn", action="store_true"), g.add_argument("--b-mn", action="store_true")
    g.add_argument("--single", action="store_true", help="one-CTA kernel only")
    g.add_argument("--epilogue", default="none", choices=["none", "gelu", "dgelu", "dropadd"])
    t = sub.add_parser("attention")
    t.add_argument("B", type=int), t.add_argument("NH", type=int), t.add_argument("S", type=int)
    t.add_argument("HD", type=int), t.add_argument("--dropout", type=float, default=0.0)
    t.add_argument("--pair", action="store_true", help="backward as the dK/dV + dQ kernel pair")
    ln = sub.add_parser("layernorm")
    ln.add_argument("rows", type=int), ln.add_argument("H", type=int)
    e = sub.add_parser("embedding")
    e.add_argument("tokens", type=int), e.add_argument("H", type=int), e.add_argument("V", type=int)
    e.add_argument("--dropout", type=float, default=0.0)
    ce = sub.add_parser("crossentropy")
    ce.add_argument("tokens", type=int), ce.add_argument("V", type=int)
    ad = sub.add_parser("adam")
    ad.add_argument("n", type=int)
    cb = sub.add_parser("convbn")
    cb.add_argument("N", type=int), cb.add_argument("HW", type=int), cb.add_argument("C", type=int)
    cb.add_argument("--filter", type=int, default=3)
    cs = sub.add_parser("colsum")
    cs.add_argument("rows", type=int), cs.add_argument("N", type=int)
    for p in (g, t, ln, e, ce, ad, cb, cs):
        p.add_argument("--warmup", type=int, default=3), p.add_argument("--iters", type=int, default=3)
    a = ap.parse_args(argv)
    {"gemm": run_gemm, "attention": run_attention, "layernorm": run_layernorm, "embedding": run_embedding,
     "crossentropy": run_crossentropy, "adam": run_adam, "convbn": run_convbn, "colsum": run_colsum}[a.kind](a)


if __name__ == "__main__":
    main()
