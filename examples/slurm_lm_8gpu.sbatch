#!/bin/bash
# One node, 8 GPUs: the 760M uTTT-MoE language model at 32K context.
#
#     sbatch examples/slurm_lm_8gpu.sbatch [extra --section.key value flags]
#
# A template: partitions, accounts and module systems differ between clusters - copy it and edit the header.
#SBATCH --job-name=uttt-lm
#SBATCH --nodes=1
#SBATCH --gres=gpu:8
#SBATCH --ntasks-per-node=1
#SBATCH --cpus-per-task=32
#SBATCH --time=48:00:00
#SBATCH --output=slurm-%j.out
set -euo pipefail
cd "${SLURM_SUBMIT_DIR:-$(pwd)}"
export NPROC_PER_NODE=8
export JOB_UUID="uttt-lm-${SLURM_JOB_ID:-$$}"
bash launch/train_lm.sh configs/lm/exp/train_760M_32k.toml configs/lm/main/760M/uttt_moe.json "run-${SLURM_JOB_ID:-local}" "$@"
