#!/bin/bash
#SBATCH --job-name=lm-engine-b200
#SBATCH --nodes=2
#SBATCH --ntasks-per-node=1
#SBATCH --gpus-per-node=8
#SBATCH --cpus-per-task=96
#SBATCH --exclusive
#SBATCH --output=logs/%x-%j.out
# One launcher task per node; launch/train.sh starts one rank per GPU under torchrun.
#   sbatch launch/slurm.sbatch configs/pretraining/llama3-8b-zero3.yml
srun --kill-on-bad-exit=1 launch/train.sh "$@"
