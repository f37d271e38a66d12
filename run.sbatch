#!/bin/bash
# SLURM template: one task per GPU, single node (8 x B200) or several nodes inside ONE NVLink
# domain (NVL72: add --segment so the allocation stays inside one domain; EP = total tasks must
# divide the expert count).  Role of the reference's run.sbatch (1 task/GPU through srun, rank
# variables exported per task), without its DeepEP build step: nothing is compiled at run time
# except `python -m moe_comms_benchmarking_b200.build`, once, before the tasks start.
#SBATCH --job-name=moe-comms-b200
#SBATCH --nodes=1
#SBATCH --ntasks-per-node=8
#SBATCH --gpus-per-node=8
#SBATCH --exclusive
#SBATCH --time=00:30:00
#SBATCH --output=moe-comms-b200-%j.out
##SBATCH --segment=2            # multi-node NVL72: keep all nodes in one NVLink domain

set -euo pipefail
cd "${SLURM_SUBMIT_DIR:-$(dirname "$0")}"
BATCHES=${BATCHES:-1,2,4,8,16,32,64,128,256,512,1024,2048,4096,8192}
IMPL=${IMPL:-all}
OUT=${OUT:-results/results_${SLURM_JOB_ID:-local}.csv}
mkdir -p "$(dirname "$OUT")"

python -m moe_comms_benchmarking_b200.build

export MASTER_ADDR=${MASTER_ADDR:-$(scontrol show hostnames "${SLURM_JOB_NODELIST:-localhost}" 2>/dev/null | head -n1 || echo 127.0.0.1)}
export MASTER_PORT=${MASTER_PORT:-29500}

LAUNCH='export RANK=$SLURM_PROCID WORLD_SIZE=$SLURM_NTASKS LOCAL_RANK=$SLURM_LOCALID; exec python run.py'
srun ${CONTAINER_IMAGE:+--container-image "$CONTAINER_IMAGE"} bash -c "$LAUNCH --impl $IMPL --validate"
srun ${CONTAINER_IMAGE:+--container-image "$CONTAINER_IMAGE"} bash -c \
  "$LAUNCH --impl $IMPL --batch-sizes $BATCHES --num-layers 88 --reps 20 --warmup 6 --timing graph --out $OUT --resume"
python plot_results.py --csv "$OUT" --out "${OUT%.csv}.png"
