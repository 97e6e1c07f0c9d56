"""Child process of tests/test_multigpu_gpu.py (one rank per GPU, launched by torch.distributed.run)."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def main():
    from superscaler_b200.data.synthetic import gpt_batch
    from superscaler_b200.ops import native
    from superscaler_b200.parallel.state import init_distributed
    from superscaler_b200.parallel.symm import SymmetricBuffer
    from superscaler_b200.runtime.trainer import Trainer
    from helpers import tiny_gpt_plan

    rank, world, local = init_distributed()
    dev = torch.device("cuda", local)
    mode = sys.argv[1]
    if mode == "allreduce":
        n = 1 << 22
        buf = SymmetricBuffer(n, torch.float32, None, dev)
        for it in range(3):
            torch.manual_seed(100 * it + rank)
            x = torch.randn(n, device=dev)
            ref = x.clone()
            dist.all_reduce(ref)
            buf.tensor.copy_(x)
            buf.allreduce_scale_(n, 1.0 / world)
            torch.cuda.synchronize()
            err = (buf.tensor - ref / world).abs().max().item()
            assert err < 1e-5, f"rank {rank} iteration {it}: max error {err} (multicast={buf.multicast_ptr != 0})"
        assert native.check_status() == 0
        if rank == 0:
            print("ALLREDUCE_OK multicast", buf.multicast_ptr != 0, flush=True)
    elif mode == "train":
        kw = dict(layers=2, seq=256, hidden=512, heads=4, head_dim=128, vocab=2048, global_bs=8, micro_bs=4)
        nd = dict(hidden_dropout=0.0, attention_dropout=0.0)
        plans = {"dp": tiny_gpt_plan(**kw, num_gpus=(world,), tp=[1]),
                 "tp": tiny_gpt_plan(**kw, num_gpus=(world,), tp=[world]),
                 "pp": tiny_gpt_plan(**kw, num_gpus=tuple([1] * world))}
        if (kw["global_bs"] // kw["micro_bs"]) % world == 0:
            from superscaler_b200.runtime.schedules import interleave_plan
            plans["pp_interleaved"] = interleave_plan(plans["pp"], 2)
        out, masters = {}, {}
        # bitwise-reproducible kernels, so that runs can be compared element by element (gradients that are pure
        # rounding noise, like the key bias of attention, otherwise differ from run to run and Adam turns them
        # into updates of full size)
        from superscaler_b200.ops import functional as F
        F.set_deterministic(True)
        for name, plan in plans.items():
            for fused in ((True, False) if name in ("dp", "tp") else (False,)):
                for shard in ((True, False) if (name == "dp" and fused) else (False,)):
                    t = Trainer(plan, rank=rank, world_size=world, model_overrides=nd, lr_warmup_steps=0,
                                fused_comm=fused, shard_optimizer=shard)
                    ls = [t.loss_value(t.train_step(gpt_batch(8, 256, 2048, seed=1))) for _ in range(3)]
                    key = f"{name}{'_fused' if fused else ''}{'_sharded' if shard else ''}"
                    out[key] = ls
                    if name == "dp":
                        assert t.optimizer.sharded == (fused and shard), key
                        sd = t.optimizer.state_dict()             # collective: gathers the slices of a sharded run
                        masters[key] = (sd["master"].clone(), sd["exp_avg_sq"].clone(), t.store.model16.clone())
                        decayed_end = t.store.wd_end
                        if t.optimizer.sharded and rank == 0:
                            print("slice", t.optimizer.shard_lo, t.optimizer.shard_hi, "wd_end", t.store.wd_end, "total",
                                  t.store.total, flush=True)
                    del t
        torch.cuda.synchronize()
        assert native.check_status() == 0
        # reduce-scatter + sharded Adam + all-gather of the bf16 weights against all-reduce + replicated Adam: the same
        # update up to the rounding of the gradient norm (summed in another order)
        assert max(abs(a - b) for a, b in zip(out["dp_fused_sharded"], out["dp_fused"])) < 1e-3, out
        diffs = [(a.float() - b.float()).abs().max().item() for a, b in zip(masters["dp_fused_sharded"], masters["dp_fused"])]
        d0 = (masters["dp_fused_sharded"][0] - masters["dp_fused"][0]).abs()
        where = (int(d0.argmax()), int((d0 > 1e-4).sum()), d0.numel())
        # Matrices (the weight-decayed front of the buffer): equal up to the rounding of the clip factor.  Biases and
        # LayerNorm parameters behind them include elements whose gradient is rounding noise around zero (a key bias
        # does not change a softmax); Adam turns that noise into steps of +-lr, so the last bit of the clip factor may
        # send such an element the other way in each of the three steps: at most 2 * 3 * lr apart.
        assert d0[:decayed_end].max().item() < 2e-4 and d0.max().item() < 6 * 1.5e-4 + 1e-5, (diffs, where)
        assert diffs[1] < 1e-4 and diffs[2] < 1e-2, (diffs, where)                           # second moment, bf16 copy
        mine = masters["dp_fused_sharded"][2].float()
        other = mine.clone()
        dist.broadcast(other, src=0)
        assert torch.equal(mine, other), "bf16 weights differ between ranks after the sharded update"
        # dp -> tp inside a stage, right at the column-parallel GEMMs: LayerNorms, embedding and the head run data
        # parallel, the attention block and the MLP tensor parallel.  The rows are then gathered INSIDE the QKV and MLP
        # up-projection kernels and their input gradients reduce-scattered by the dgrad kernel; with SSB_FUSED_GATHER=0
        # the relayout engine moves them with NCCL instead.  Both must train like the data-parallel run.
        from superscaler_b200.models.gpt import gpt_op_names
        names = gpt_op_names(kw["layers"])
        mixed = tiny_gpt_plan(**kw, num_gpus=(world,), tp=[1])
        mixed["model_parallel_size_of_each_op"] = [[world if (("attention" in n and "post" not in n) or "MLP-GEMM" in n
                                                                or "MLP-gelu" in n) else 1 for n in names]]
        mixed["data_parallel_size_of_each_op"] = [[world // t for t in mixed["model_parallel_size_of_each_op"][0]]]
        mixed["resharding_stages"] = [True]
        for fused_gather in ("1", "0"):
            os.environ["SSB_FUSED_GATHER"] = fused_gather
            t = Trainer(mixed, rank=rank, world_size=world, model_overrides=nd, lr_warmup_steps=0, fused_comm=True)
            out[f"mixed_gather{fused_gather}"] = [t.loss_value(t.train_step(gpt_batch(8, 256, 2048, seed=1))) for _ in range(3)]
            if fused_gather == "1":
                used = [type(o).__name__ for o in t.stage.ops if getattr(o, "accepts_dealt_out_rows", lambda: False)()]
                assert used, "no op of the mixed plan takes dealt-out rows"
            del t
        os.environ.pop("SSB_FUSED_GATHER")
        torch.cuda.synchronize()
        assert native.check_status() == 0
        assert max(abs(a - b) for a, b in zip(out["mixed_gather1"], out["mixed_gather0"])) < 2e-3, out
        base = out["dp"]
        for k, v in out.items():
            assert all(x == x for x in v) and v[-1] < v[0], (k, v)
            assert max(abs(a - b) for a, b in zip(base, v)) < 5e-2, (k, v, base)
        if rank == 0:
            print("TRAIN_OK", {k: [round(x, 4) for x in v] for k, v in out.items()}, "sharded vs replicated", diffs,
                  flush=True)
    elif mode == "gemm_ar":
        from superscaler_b200.ops import functional as F
        from superscaler_b200.parallel.symm import FusedTPContext
        ctx = FusedTPContext(None, 4096, 2048, dev)
        use_mc = [False]
        cases = [(1000, 512, 256, False, 0.0), (4096, 2048, 1024, False, 0.1), (2048, 1024, 512, True, 0.0),
                 (256, 256, 64, False, 0.0), (4096, 2048, 1024, True, 0.1)]
        worst = 0.0
        for mc in use_mc:
            for rep in range(2):
                for (M, N, K, b_mn, pdrop) in cases:
                    g = torch.Generator(device=dev).manual_seed(1000 * rank + M + N + rep)
                    x = (torch.randn(M, K, device=dev, generator=g) * 0.5).bfloat16()
                    w = (torch.randn((K, N) if b_mn else (N, K), device=dev, generator=g) * 0.1).bfloat16()
                    g2 = torch.Generator(device=dev).manual_seed(7 + rep)       # same on every rank
                    bias = torch.randn(N, device=dev, generator=g2).bfloat16()
                    res = torch.randn(M, N, device=dev, generator=g2).bfloat16()
                    out = ctx.linear_allreduce(x, w, b_mn=b_mn, bias=bias, residual=res, dropout_p=pdrop, seed=99)
                    # unfused path with this framework's own kernels + NCCL
                    y = F.gemm(x, w, b_mn=b_mn, out_dtype=torch.float32)
                    dist.all_reduce(y)
                    ref = F.bias_dropout_add(y.bfloat16(), bias, res, pdrop, 99)
                    torch.cuda.synchronize()
                    err = (out.float() - ref.float()).abs().max().item()
                    scale = ref.float().abs().max().item()
                    worst = max(worst, err / scale)
                    assert err / scale < 2e-2, f"rank {rank} mc={mc} case {(M, N, K, b_mn, pdrop)}: err {err} scale {scale}"
                    if pdrop > 0:   # identical dropout masks: zeros of (out - res) coincide
                        z1 = (out.float() - res.float()) == 0
                        z2 = (ref.float() - res.float()) == 0
                        assert (z1 != z2).float().mean().item() < 1e-3
        assert native.check_status() == 0
        gathered = [None] * world
        dist.all_gather_object(gathered, float(out.float().sum().item()))
        assert all(abs(v - gathered[0]) < 1e-3 * max(1.0, abs(gathered[0])) for v in gathered), gathered
        if rank == 0:
            print("GEMM_AR_OK worst rel err", round(worst, 5), flush=True)
    elif mode == "gemm_rs":
        # GEMM -> reduce-scatter form of the fused kernel against GEMM + NCCL reduce_scatter, interleaved with the
        # all-reduce form on the same scratch (the "consumed" hand-shake keeps a fast rank from overwriting partials
        # an owner still reads)
        from superscaler_b200.ops import functional as F
        from superscaler_b200.parallel.symm import FusedTPContext
        ctx = FusedTPContext(None, 4096, 2048, dev)
        worst = 0.0
        for rep in range(3):
            for (M, N, K, b_mn) in [(256 * world, 512, 256, False), (4096, 2048, 1024, True), (1024, 1024, 512, False)]:
                g = torch.Generator(device=dev).manual_seed(31 * rank + M + N + rep)
                x = (torch.randn(M, K, device=dev, generator=g) * 0.5).bfloat16()
                w = (torch.randn((K, N) if b_mn else (N, K), device=dev, generator=g) * 0.1).bfloat16()
                out = ctx.linear_reduce_scatter(x, w, b_mn=b_mn)
                y = F.gemm(x, w, b_mn=b_mn, out_dtype=torch.float32)
                ref = torch.empty(M // world, N, device=dev, dtype=torch.float32)
                dist.reduce_scatter_tensor(ref, y)
                full = ctx.linear_allreduce(x, w, b_mn=b_mn)          # the other form right behind it, same scratch
                dist.all_reduce(y)
                torch.cuda.synchronize()
                scale = ref.abs().max().item()
                err = (out.float() - ref).abs().max().item() / scale
                err2 = (full.float() - y).abs().max().item() / y.abs().max().item()
                worst = max(worst, err, err2)
                assert err < 2e-2 and err2 < 2e-2, f"rank {rank} case {(M, N, K, b_mn)} rep {rep}: {err} {err2}"
        assert native.check_status() == 0
        if rank == 0:
            print("GEMM_RS_OK worst rel err", round(worst, 5), flush=True)
    elif mode == "ag_gemm":
        from superscaler_b200.ops import functional as F
        from superscaler_b200.parallel.symm import FusedTPContext
        ctx = FusedTPContext(None, 256, 256, dev)
        ctx.enable_allgather(2048 * world, 1024)
        worst = 0.0
        for rep in range(3):
            for (rows, N, K, act) in [(128, 256, 64, 0), (2048, 1024, 1024, 1), (512, 776 // 8 * 8, 256, 0), (1024, 4096, 512, 1)]:
                g = torch.Generator(device=dev).manual_seed(50 * rank + rows + rep)
                x = torch.randn(rows, K, device=dev, generator=g).bfloat16()
                g2 = torch.Generator(device=dev).manual_seed(3 + rep)          # same on every rank
                w = (torch.randn(N, K, device=dev, generator=g2) * 0.05).bfloat16()
                bias = torch.randn(N, device=dev, generator=g2).bfloat16()
                out = ctx.allgather_linear(x, w, bias=bias, act=act)
                full = [torch.empty_like(x) for _ in range(world)]
                dist.all_gather(full, x)
                ref = F.gemm(torch.cat(full, 0), w, bias=bias, act=act)
                torch.cuda.synchronize()
                err = (out.float() - ref.float()).abs().max().item()
                worst = max(worst, err)
                assert err <= 1e-2 * ref.float().abs().max().item(), f"rank {rank} case {(rows, N, K, act)} rep {rep}: max err {err}"
        assert native.check_status() == 0
        if rank == 0:
            print("AG_GEMM_OK", worst, flush=True)
    # guard words around the symmetric buffers (placed when SSB_CANARIES=1; none otherwise) must be intact
    from superscaler_b200.parallel.guards import REGISTRY
    torch.cuda.synchronize()
    damaged = REGISTRY.check()
    assert not damaged, damaged
    if os.environ.get("SSB_CANARIES") == "1":
        assert REGISTRY.buffers, "SSB_CANARIES=1 but no guarded buffer was allocated"
        if rank == 0:
            print("GUARDS_OK", len(REGISTRY.buffers), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
