#!/usr/bin/env bash
# Train a language model:  NPROC_PER_NODE=8 bash launch/train_lm.sh [--dry-run] <job.toml> <model.json> [job_name] [flags]
set -euo pipefail
ROOT="$(cd "$(dirname "$0")/.." && pwd)"
cd "$ROOT"
exec "${PYTHON:-python3}" -m uttt_b200.launch lm "$@"
