#!/bin/bash
# Search, grid-planned baseline, three training iterations of every saved plan, result tables and figures for the
# three models at the "small" experiment size (one node, 4 GPUs).  Other sizes: MODE=large or MODE=scale.
set -euo pipefail
MODE=${MODE:-small}
python -m superscaler_b200.experiments all --mode "$MODE" --results "${RESULTS:-./logs}" "$@"
