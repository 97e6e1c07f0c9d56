#!/bin/bash
# One node of a training job from a plan JSON (any of the three models: the plan names its model).  Start it once per
# node with the same plan and MASTER_ADDR / MASTER_PORT; NODE_RANK counts the nodes from 0.
#
#   examples/run_node.sh plans/gpt_1_3B_8gpu_b200.json [log_dir] [extra runtime.pretrain flags ...]
#
# Environment: NNODES (1), GPUS_PER_NODE (all visible GPUs), NODE_RANK (0), MASTER_ADDR (127.0.0.1), MASTER_PORT (7000),
# TRAIN_ITERS (3).  The per-rank CSVs of the last iteration land in <log_dir>/csv/ (the files
# `python -m superscaler_b200.utils.results` and `superscaler_b200.experiments collect` read); the full log of this
# node in <log_dir>/full_log_<plan>_rank<NODE_RANK>_<time>.
set -euo pipefail
PLAN=${1:?plan JSON}; shift
LOG_PATH=${1:-./logs}/; [ $# -gt 0 ] && shift
NNODES=${NNODES:-1}
GPUS_PER_NODE=${GPUS_PER_NODE:-$(python -c 'import torch; print(max(1, torch.cuda.device_count()))')}
NODE_RANK=${NODE_RANK:-0}
MASTER_ADDR=${MASTER_ADDR:-127.0.0.1}
MASTER_PORT=${MASTER_PORT:-7000}
mkdir -p "${LOG_PATH}csv"
NAME=$(basename "$PLAN" .json)
NOW=$(date '+%Y-%m-%d-%H-%M-%S')
python -m torch.distributed.run --nnodes "$NNODES" --nproc-per-node "$GPUS_PER_NODE" --node-rank "$NODE_RANK" \
    --master-addr "$MASTER_ADDR" --master-port "$MASTER_PORT" \
    -m superscaler_b200.runtime.pretrain \
    --flexpipe-config "$PLAN" \
    --train-iters "${TRAIN_ITERS:-3}" \
    --eval-iters 0 \
    --lr-decay-iters 320000 \
    --lr 0.00015 \
    --lr-decay-style cosine \
    --min-lr 1.0e-5 \
    --weight-decay 1e-2 \
    --clip-grad 1.0 \
    --lr-warmup-fraction .01 \
    --log-interval 1 \
    --log-path "$LOG_PATH" \
    "$@" 2>&1 | tee "${LOG_PATH}full_log_${NAME}_rank${NODE_RANK}_${NOW}"
