#!/bin/bash
# Two nodes of 8 GPUs: a view-synthesis configuration at 8 scenes per GPU (total batch 128).
#
#     sbatch examples/slurm_nvs_multinode.sbatch configs/nvs/capacity/obj/uttt_moe_e64a1.yaml \
#         -s training.batch_size_per_gpu 8
#
# Only the total number of GPUs enters the batch size; change it and training.batch_size_per_gpu together, or the
# trainer stops at its batch-size check.  A template: copy it and edit the header for your cluster.
#SBATCH --job-name=uttt-nvs-16gpu
#SBATCH --nodes=2
#SBATCH --gres=gpu:8
#SBATCH --ntasks-per-node=1
#SBATCH --cpus-per-task=32
#SBATCH --time=48:00:00
#SBATCH --output=slurm-%j.out
set -euo pipefail
CONFIG="${1:?usage: sbatch slurm_nvs_multinode.sbatch <config.yaml> [-s overrides]}"
shift || true
cd "${SLURM_SUBMIT_DIR:-$(pwd)}"
# The launcher reads the usual PyTorch variables; SLURM does not set them, so they are derived from the allocation.
# WORLD_SIZE counts processes over all nodes; setting MASTER_PORT is what selects the multi-node rendezvous.
export NPROC_PER_NODE=8
export JOB_UUID="uttt-nvs-${SLURM_JOB_ID:-$$}"
export MASTER_ADDR="$(scontrol show hostnames "${SLURM_JOB_NODELIST}" | head -n1)"
export MASTER_PORT="${MASTER_PORT:-29500}"
export WORLD_SIZE=$(( SLURM_JOB_NUM_NODES * NPROC_PER_NODE ))
# one task per node: srun starts the launcher everywhere, torchrun starts the workers of its node
srun --ntasks-per-node=1 bash -c 'export NODE_RANK=${SLURM_NODEID}; bash launch/train_nvs.sh "$@"' _ "${CONFIG}" "$@"
