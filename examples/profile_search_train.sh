#!/bin/bash
# One node with N GPUs: profile -> search -> train, the three steps of the workflow, for any of the three models.
# Usage: examples/profile_search_train.sh <gpt|t5|resnet> <model size> <num_gpus> [work_dir] [num_layers]
#   gpt 350M | 1_3B | 2_6B | 6_7B | 13B, t5 770M | 3B | 6B | 11B | 22B, resnet 500M | 1B | 2B | 4B | 6_8B | 13B
# The optional num_layers trains a deeper or shallower GPT / T5 of the same width ("scale-layer" runs).
set -euo pipefail
MODEL=${1:?model}; SIZE=${2:?size}; N=${3:-8}
WORK=${4:-./runs/${MODEL}_${SIZE}_${N}gpu}
LAYERS=${5:-}
case $MODEL in
  gpt)    GBS=512; PER_GPU="1 2 4 8 16" ;;
  t5)     GBS=512; PER_GPU="1 2 4 8 16 32" ;;
  resnet) GBS=768; PER_GPU="16 32 48 64" ;;
  *) echo "unknown model $MODEL"; exit 2 ;;
esac
DB=$WORK/profiled-time/
mkdir -p "$DB" "$WORK/plans" "$WORK/logs"
RUN="python -m torch.distributed.run --nnodes=1 --master-addr 127.0.0.1 --master-port 29500"
EXTRA=""; if [ -n "$LAYERS" ]; then EXTRA="--num-layers $LAYERS"; fi

# 1. profile: op tables for every tensor-parallel degree up to N, then collectives and p2p bandwidth
tp=1
while [ $tp -le $N ]; do
  $RUN --nproc-per-node $tp -m superscaler_b200.profiler.op_profiler --model-name $MODEL --model-size $SIZE \
      --prof-tp-size $tp --prof-mbs-list $PER_GPU --prof-path "$DB"
  tp=$((tp * 2))
done
if [ $N -gt 1 ]; then
  if [ $MODEL != t5 ]; then   # T5 plans never reshard inside a stage, so no collective table is needed
    $RUN --nproc-per-node $N -m superscaler_b200.profiler.comm_profiler --model-name $MODEL --model-size $SIZE --prof-path "$DB"
  fi
  $RUN --nproc-per-node 2 -m superscaler_b200.profiler.p2p_profiler --prof-path "$DB"
fi

# 2. search (CPU only); micro-batch candidates: every per-GPU size times 1, 2, 4 ... N that divides the global batch
MBS=$(python - "$GBS" "$N" $PER_GPU <<'PY'
import sys
gbs, n, per = int(sys.argv[1]), int(sys.argv[2]), [int(x) for x in sys.argv[3:]]
cands, k = set(), 1
while k <= n:
    cands.update(p * k for p in per if gbs % (p * k) == 0)
    k *= 2
print(" ".join(map(str, sorted(cands))))
PY
)
python -m superscaler_b200.search.search --model-name $MODEL --model-size $SIZE --global-batch-size $GBS \
    --micro-batch-size $MBS --max-tp $N --num-nodes 1 --num-gpus-per-node $N --memory-limit 170000 \
    --profiled-time-path "$DB" --config-save-path "$WORK/plans/" --log-path "$WORK/logs/" --shapes b200 \
    --max-num-hops 7 --time-budget-total 200 $EXTRA
PLAN=$(python - "$WORK" "$MODEL" "$SIZE" <<'PY'
import csv, glob, sys
work, model, size = sys.argv[1:4]
best = None
for f in glob.glob(f"{work}/plans/csv/info_{model}_{size}_*stages_*.csv"):
    t = max(float(r[1]) for r in list(csv.reader(open(f)))[1:])
    if best is None or t < best[0]:
        best = (t, f.replace("/csv/info_", "/").replace(".csv", ".json"))
print(best[1])
PY
)
echo "best plan: $PLAN"

# 3. train 3 iterations from the plan; per-rank CSVs under $WORK/logs/csv, then throughput and prediction error
$RUN --nproc-per-node $N -m superscaler_b200.runtime.pretrain --flexpipe-config "$PLAN" --train-iters 3 --log-path "$WORK/logs"
python -m superscaler_b200.utils.results --log-path "$WORK/logs"
