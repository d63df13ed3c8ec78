#!/usr/bin/env bash
# Per-token-loss evaluation of a trained language model:
#
#   NPROC_PER_NODE=8 bash launch/eval_ptl.sh configs/lm/exp/eval_ptl.toml /path/to/hf_model_dir [--section.key value ...]
#
# The checkpoint is a HF-style folder (config.json + weights), written by `python -m uttt_b200.utils.convert dcp-to-hf`.
# The job file names the 32K-token shards (training.data_files) and the lm-head chunk ([eval] lm_head_chunk_size);
# set training.steps to rows / (batch_size x GPUs).  Result: <job.dump_folder>/<save_prefix>_loss_per_token_position.json;
# reduce it with `python -m uttt_b200.eval.ptl summarize FILE.json`.
set -euo pipefail
JOB="${1:?usage: eval_ptl.sh <eval_ptl.toml> <hf_checkpoint_dir> [extra flags]}"
CKPT="${2:?usage: eval_ptl.sh <eval_ptl.toml> <hf_checkpoint_dir> [extra flags]}"
ROOT="$(cd "$(dirname "$0")/.." && pwd)"
cd "$ROOT"
exec torchrun --standalone --local-addr 127.0.0.1 --nproc_per_node="${NPROC_PER_NODE:-8}" \
  -m uttt_b200.eval.ptl --job.config_file "$JOB" --checkpoint.load_path "$CKPT" "${@:3}"
