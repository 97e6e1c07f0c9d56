"""Vision-transformer entry point, beside the reference's runtime/pretrain_gpt.py / pretrain_t5.py /
pretrain_resnet.py (the reference's tree holds the ViT data pipeline, runtime/megatron/data/vit_dataset.py, and its
flags, but no ViT entry point; here it is an op-list model): trains the plan given by --flexpipe-config, which must be a vit plan (`"model_name": "vit"`, the GPT
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
