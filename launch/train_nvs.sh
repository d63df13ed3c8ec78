#!/usr/bin/env bash
# Train a view-synthesis model:  NPROC_PER_NODE=4 bash launch/train_nvs.sh [--dry-run] <config.yaml> [-s key value ...]
set -euo pipefail
ROOT="$(cd "$(dirname "$0")/.." && pwd)"
cd "$ROOT"
exec "${PYTHON:-python3}" -m uttt_b200.launch nvs "$@"
