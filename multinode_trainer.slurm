#!/bin/bash
#SBATCH --job-name=torchtitan_b200
#SBATCH --ntasks-per-node=1
#SBATCH --gpus-per-node=8
#SBATCH --cpus-per-task=96
#SBATCH --exclusive
#SBATCH --output=slurm-%j.out
#
# Training over several nodes under Slurm: one launcher agent per node, one process per GPU.
#
#   sbatch --nodes 4 multinode_trainer.slurm --training.steps 1000
#   MODULE=qwen3 CONFIG=qwen3_30b_a3b sbatch --nodes 2 multinode_trainer.slurm --parallelism.expert_parallel_degree 8
#
# Inside a node the framework's own peer-memory collectives (FSDP transport, fused tensor-parallel GEMMs, expert
# exchange) run over NVLink; a parallel dimension whose groups span nodes takes NCCL. Tensor, expert and shard
# dimensions come last in the rank order, so with 8 GPUs per node any tp x shard (or tp x ep) product up to 8 stays on
# NVLink, and data_parallel_replicate / pipeline stages go across nodes.
# `python -m torchtitan_b200.experiments.autoparallel.planner --module M --config C --ngpu N` proposes a layout.
#
# Fabric settings are site-specific: export NCCL_SOCKET_IFNAME / NCCL_IB_HCA (or your provider's variables) before sbatch.

set -euo pipefail

: "${MODULE:=llama3}" "${CONFIG:=llama3_debugmodel}" "${GPUS_PER_NODE:=8}" "${RDZV_PORT:=29500}"
rendezvous_host=$(scontrol show hostnames "$SLURM_JOB_NODELIST" | head -n 1)
echo "rendezvous at $rendezvous_host:$RDZV_PORT, $SLURM_JOB_NUM_NODES node(s) x $GPUS_PER_NODE GPUs, $MODULE / $CONFIG"

export PYTORCH_ALLOC_CONF="expandable_segments:True" PYTHONFAULTHANDLER=1
export NCCL_DEBUG="${NCCL_DEBUG:-WARN}" LOGLEVEL="${LOGLEVEL:-INFO}"

srun python3 -m torch.distributed.run \
    --nnodes "$SLURM_JOB_NUM_NODES" --nproc_per_node "$GPUS_PER_NODE" \
    --rdzv_backend c10d --rdzv_id "$SLURM_JOB_ID" --rdzv_endpoint "$rendezvous_host:$RDZV_PORT" \
    -m torchtitan_b200.train --module "$MODULE" --config "$CONFIG" "$@"
