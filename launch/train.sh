#!/bin/bash
# Launches `lm_engine_b200.train` (or .distill / .unshard, second argument) on every GPU of this node, or of all the
# nodes of a Slurm / LSF allocation.  One process per GPU; rendezvous over the first node of the allocation.
#   launch/train.sh configs/pretraining/llama3-8b-zero3.yml [train|distill|unshard]
set -euo pipefail
CONFIG=${1:?usage: launch/train.sh <config.yml> [train|distill|unshard]}
ENTRY=${2:-train}

if [[ -n "${SLURM_JOB_NODELIST:-}" ]]; then
    MASTER_ADDRESS=$(scontrol show hostnames "$SLURM_JOB_NODELIST" | head -n 1)
    NNODES=${SLURM_NNODES}
    NODE_RANK=${SLURM_NODEID}
    MASTER_PORT=$((20000 + SLURM_JOB_ID % 20000))
elif [[ -n "${LSB_MCPU_HOSTS:-}" ]]; then
    MASTER_ADDRESS=$(echo ${LSB_MCPU_HOSTS} | tr ' ' '\n' | head -n 1)
    NNODES=$(echo ${LSB_MCPU_HOSTS} | tr ' ' '\n' | sed 'n; d' | wc -w)
    NODE_RANK=$(($(echo ${LSB_MCPU_HOSTS} | tr ' ' '\n' | sed 'n; d' | grep -n -m1 "$(hostname -s)" | cut -d: -f1) - 1))
    MASTER_PORT=$((20000 + LSB_JOBID % 20000))
else
    MASTER_ADDRESS=127.0.0.1
    NNODES=1
    NODE_RANK=0
    MASTER_PORT=${MASTER_PORT:-29500}
fi
GPUS_PER_NODE=${GPUS_PER_NODE:-$(nvidia-smi -L | wc -l)}

# NVLink / NVSwitch domain: let NCCL use in-switch reductions; keep the tokenizer library single threaded
export NCCL_NVLS_ENABLE=${NCCL_NVLS_ENABLE:-1}
export TOKENIZERS_PARALLELISM=false
export OMP_NUM_THREADS=${OMP_NUM_THREADS:-8}

exec python -m torch.distributed.run \
    --nnodes="$NNODES" --node_rank="$NODE_RANK" --nproc_per_node="$GPUS_PER_NODE" \
    --rdzv_id=101 --rdzv_backend=c10d --rdzv_endpoint="$MASTER_ADDRESS:$MASTER_PORT" \
    -m "lm_engine_b200.$ENTRY" --config "$CONFIG"
