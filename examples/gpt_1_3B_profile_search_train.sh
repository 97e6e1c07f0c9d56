#!/bin/bash
# GPT-3 1.3B on one node with N GPUs: profile -> search -> train, the three steps of the workflow.
# Usage: examples/gpt_1_3B_profile_search_train.sh <num_gpus> [work_dir]
set -euo pipefail
N=${1:-8}
WORK=${2:-./runs/gpt_1_3B_${N}gpu}
DB=$WORK/profiled-time/
mkdir -p "$DB" "$WORK/plans" "$WORK/logs"
RUN="python -m torch.distributed.run --nnodes=1 --master-addr 127.0.0.1 --master-port 29500"

# 1. profile: op tables for every tensor-parallel degree up to N, then collectives and p2p bandwidth
tp=1
while [ $tp -le $N ]; do
  $RUN --nproc-per-node $tp -m superscaler_b200.profiler.op_profiler --model-name gpt --model-size 1_3B \
      --prof-tp-size $tp --prof-mbs-list 1 2 4 8 16 --prof-path "$DB"
  tp=$((tp * 2))
done
if [ $N -gt 1 ]; then
  $RUN --nproc-per-node $N -m superscaler_b200.profiler.comm_profiler --model-name gpt --model-size 1_3B --prof-path "$DB"
  $RUN --nproc-per-node 2 -m superscaler_b200.profiler.p2p_profiler --prof-path "$DB"
fi

# 2. search (CPU only); micro-batch candidates up to 16 samples per GPU
MBS="1 2 4 8 16"; m=32; while [ $m -le $((16 * N)) ]; do MBS="$MBS $m"; m=$((m * 2)); done
python -m superscaler_b200.search.search --model-name gpt --model-size 1_3B --global-batch-size 512 \
    --micro-batch-size $MBS --max-tp $N --num-nodes 1 --num-gpus-per-node $N --memory-limit 170000 \
    --profiled-time-path "$DB" --config-save-path "$WORK/plans/" --log-path "$WORK/logs/" --shapes b200 \
    --max-num-hops 7 --time-budget-total 200
PLAN=$(python - "$WORK" <<'PY'
import csv, glob, sys
work = sys.argv[1]
best = None
for f in glob.glob(f"{work}/plans/csv/info_gpt_1_3B_*stages_*.csv"):
    t = max(float(r[1]) for r in list(csv.reader(open(f)))[1:])
    if best is None or t < best[0]:
        best = (t, f.replace("/csv/info_", "/").replace(".csv", ".json"))
print(best[1])
PY
)
echo "best plan: $PLAN"

# 3. train 3 iterations from the plan; per-rank CSVs under $WORK/logs/csv
$RUN --nproc-per-node $N -m superscaler_b200.runtime.pretrain --flexpipe-config "$PLAN" --train-iters 3 --log-path "$WORK/logs"
python -m superscaler_b200.utils.results --log-path "$WORK/logs"
