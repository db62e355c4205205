#!/bin/bash
# Multi-node training under Slurm: one torchrun agent per node, one process per GPU.
#
#   sbatch --nodes 4 multinode_trainer.slurm --training.steps 1000
#   MODULE=qwen3 CONFIG=qwen3_30b_a3b sbatch --nodes 2 multinode_trainer.slurm --parallelism.expert_parallel_degree 8
#
# Inside a node the framework's own peer-memory collectives (FSDP transport, fused tensor-parallel GEMMs, expert
# exchange) run over NVLink; a parallel dimension whose groups span nodes takes NCCL. Keep tensor, expert and (where it
# fits) shard groups inside a node: they come last in the rank order, so with 8 GPUs per node any product
# tp x ep-or-shard <= 8 stays on NVLink and data_parallel_replicate / pipeline stages go across nodes.

#SBATCH --job-name=torchtitan_b200
#SBATCH --ntasks-per-node=1
#SBATCH --gpus-per-node=8
#SBATCH --cpus-per-task=96
#SBATCH --exclusive
#SBATCH --output=slurm-%j.out

set -euo pipefail

nodes=( $(scontrol show hostnames "$SLURM_JOB_NODELIST") )
head_node=${nodes[0]}
head_node_ip=$(srun --nodes=1 --ntasks=1 -w "$head_node" hostname --ip-address | awk '{print $1}')
echo "head node: $head_node ($head_node_ip), ${#nodes[@]} node(s)"

export LOGLEVEL=${LOGLEVEL:-INFO}
export NCCL_DEBUG=${NCCL_DEBUG:-WARN}
export PYTHONFAULTHANDLER=1
export PYTORCH_ALLOC_CONF="expandable_segments:True"
# fabric settings are site-specific: set NCCL_SOCKET_IFNAME / NCCL_IB_HCA (or the EFA variables) for your cluster here

MODULE=${MODULE:-"llama3"}
CONFIG=${CONFIG:-"llama3_debugmodel"}
GPUS_PER_NODE=${GPUS_PER_NODE:-8}

srun python3 -m torch.distributed.run --nnodes "${#nodes[@]}" --nproc_per_node "$GPUS_PER_NODE" \
    --rdzv_id "$SLURM_JOB_ID" --rdzv_backend c10d --rdzv_endpoint "$head_node_ip:29500" \
    -m torchtitan_b200.train --module "$MODULE" --config "$CONFIG" "$@"
