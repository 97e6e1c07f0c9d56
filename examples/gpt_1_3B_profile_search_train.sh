#!/bin/bash
# GPT-3 1.3B on one node with N GPUs: profile -> search -> train.
# Usage: examples/gpt_1_3B_profile_search_train.sh <num_gpus> [work_dir]
set -euo pipefail
exec "$(dirname "$0")/profile_search_train.sh" gpt 1_3B "${1:-8}" ${2:+"$2"}
