"""BERT entry point, beside the reference's runtime/pretrain_gpt.py / pretrain_t5.py / pretrain_resnet.py (the
reference's tree holds BERT's data pipeline, runtime/megatron/data/bert_dataset.py, but no BERT entry point; here BERT
is an op-list model like the others): trains the plan given by --flexpipe-config, which must be a bert plan
(`"model_name": "bert"` with the GPT plan keys).  Synthetic two-segment batches by default; `--data-path <prefix>
--vocab-file vocab.txt` trains on a sentence corpus written by `python -m superscaler_b200.data.preprocess
--split-sentences`.  All three entry points share one implementation (superscaler_b200.runtime.pretrain); launch one rank per GPU:

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 examples/pretrain_bert.py \
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
        if name != "bert":
            sys.exit(f"pretrain_bert.py was given a {name} plan")
    pretrain.main(argv)
