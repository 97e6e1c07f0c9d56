"""Counterpart of the reference's runtime/pretrain_vit.py (inherited there from Megatron-LM as a module tree; here an
op-list model): trains the plan given by --flexpipe-config, which must be a vit plan (`"model_name": "vit"`, the GPT
plan keys for the layers, plus `image_size`, `patch_dim`, `num_classes`).  Synthetic images by default; `--data-path
<folder>` trains on `folder/train/<class>/<image>` with the AutoAugment pipeline.  All three entry points share one implementation (superscaler_b200.runtime.pretrain); launch one rank per GPU:

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 examples/pretrain_vit.py \
        --flexpipe-config plan.json --train-iters 3 --log-path logs/
"""
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from superscaler_b200.runtime import pretrain  # noqa: E402

if __name__ == "__main__":
    argv = sys.argv[1:]
    if "--flexpipe-config" in argv:
        with open(argv[argv.index("--flexpipe-config") + 1]) as f:
            name = json.load(f)["model_name"]
        if name != "vit":
            sys.exit(f"pretrain_vit.py was given a {name} plan")
    pretrain.main(argv)
