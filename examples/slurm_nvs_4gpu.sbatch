#!/bin/bash
# One node, 4 GPUs: a view-synthesis configuration with 32 scenes per GPU (total batch 128).
#
#     sbatch examples/slurm_nvs_4gpu.sbatch configs/nvs/ownership/obj/uttt_moe_e64a1.yaml [-s key value ...]
#
# A template: copy it and edit the header for your cluster.  With another GPU count change
# training.batch_size_per_gpu as well, or the trainer stops at its batch-size check.
#SBATCH --job-name=uttt-nvs
#SBATCH --nodes=1
#SBATCH --gres=gpu:4
#SBATCH --ntasks-per-node=1
#SBATCH --cpus-per-task=16
#SBATCH --time=24:00:00
#SBATCH --output=slurm-%j.out
set -euo pipefail
CONFIG="${1:?usage: sbatch slurm_nvs_4gpu.sbatch <config.yaml> [-s overrides]}"
shift || true
cd "${SLURM_SUBMIT_DIR:-$(pwd)}"
export NPROC_PER_NODE=4
export JOB_UUID="uttt-nvs-${SLURM_JOB_ID:-$$}"
bash launch/train_nvs.sh "${CONFIG}" "$@"
