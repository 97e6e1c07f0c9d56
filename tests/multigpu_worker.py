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
        out = {}
        for name, plan in plans.items():
            for fused in ((True, False) if name == "dp" else (False,)):
                t = Trainer(plan, rank=rank, world_size=world, model_overrides=nd, lr_warmup_steps=0, fused_comm=fused)
                ls = [t.loss_value(t.train_step(gpt_batch(8, 256, 2048, seed=1))) for _ in range(3)]
                out[f"{name}{'_fused' if fused else ''}"] = ls
                del t
        torch.cuda.synchronize()
        assert native.check_status() == 0
        base = out["dp"]
        for k, v in out.items():
            assert all(x == x for x in v) and v[-1] < v[0], (k, v)
            assert max(abs(a - b) for a, b in zip(base, v)) < 5e-2, (k, v, base)
        if rank == 0:
            print("TRAIN_OK", {k: [round(x, 4) for x in v] for k, v in out.items()}, flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
