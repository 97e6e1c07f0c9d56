#!/bin/bash
# Keeps a GPT training job alive across rank failures: the job runs with the heartbeat monitor; when it leaves with
# exit code 3 (a peer failed or went silent) the plan is searched again for the GPUs that are still usable and the run
# continues from the last checkpoint, whose shards are merged and re-sliced for the new plan.
# Usage: examples/elastic_train.sh <profiled-time-path> <work_dir> <train_iters> <gpu counts to fall back through...>
#   e.g. examples/elastic_train.sh profiled-time-b200/ runs/elastic 1000 8 4 2 1
set -uo pipefail
DB=${1:?database}; WORK=${2:?work dir}; ITERS=${3:?iterations}; shift 3
mkdir -p "$WORK/plans" "$WORK/logs" "$WORK/ckpt"
RUN="python -m torch.distributed.run --nnodes=1 --master-addr 127.0.0.1 --master-port 29500"
LOAD=""
for N in "$@"; do
  MBS=$(python - "$N" <<'PY'
import sys
n = int(sys.argv[1])
print(" ".join(str(m * k) for k in (1, 2, 4, 8) if k <= n for m in (1, 2, 4, 8, 16) if 512 % (m * k) == 0))
PY
)
  python -m superscaler_b200.search.search --model-name gpt --model-size 1_3B --global-batch-size 512 \
      --micro-batch-size $(echo $MBS | tr ' ' '\n' | sort -nu | tr '\n' ' ') --max-tp "$N" --num-nodes 1 \
      --num-gpus-per-node "$N" --memory-limit 170000 --profiled-time-path "$DB" --config-save-path "$WORK/plans/" \
      --log-path "$WORK/logs/" --config-suffix "n$N" --shapes b200 --max-num-hops 7 --time-budget-total 60 > "$WORK/logs/search_n$N.log" 2>&1
  PLAN=$(python - "$WORK" "$N" <<'PY'
import csv, glob, sys
work, n = sys.argv[1:3]
best = None
for f in glob.glob(f"{work}/plans/csv/info_gpt_1_3B_*stages_n{n}.csv"):
    t = max(float(r[1]) for r in list(csv.reader(open(f)))[1:])
    if best is None or t < best[0]:
        best = (t, f.replace("/csv/info_", "/").replace(".csv", ".json"))
print(best[1])
PY
)
  echo "training on $N GPUs with $PLAN $LOAD"
  $RUN --nproc-per-node "$N" -m superscaler_b200.runtime.pretrain --flexpipe-config "$PLAN" --train-iters "$ITERS" \
      --save "$WORK/ckpt" --save-interval 50 --health-check --log-path "$WORK/logs" $LOAD
  rc=$?
  if [ $rc -eq 0 ]; then echo "finished"; exit 0; fi
  echo "run on $N GPUs ended with exit code $rc; falling back"
  if [ -f "$WORK/ckpt/latest_checkpointed_iteration.txt" ]; then LOAD="--load $WORK/ckpt --load-resharded"; fi
done
echo "no GPU count left to fall back to"; exit 1
