#!/bin/bash
# Tuning pipeline for one shape (reference: run.sh:17-66):
#   profile the GEMM tiles -> measure the bandwidth curves -> search -> speed test.
# usage: ./run.sh M N K comm_op [devices]      e.g. ./run.sh 4096 8192 1024 all_reduce 0,1,2,3,4,5,6,7
# K is the per-rank K.  POINTS / REPS shorten the bandwidth curves (default: the reference's 36 sizes, 200 repetitions);
# FLASHOVERLAP_CONFIG_DIR moves the config directory.
set -euo pipefail
M=${1:-4096}; N=${2:-8192}; K=${3:-1024}; COMM_OP=${4:-all_reduce}; DEVICES=${5:-0,1}
POINTS=${POINTS:-36}; REPS=${REPS:-200}
if [ -n "${FLASH_DEBUG:-}" ]; then set -x; fi
NUM=$(echo "$DEVICES" | awk -F',' '{print NF}')
FIRST=${DEVICES%%,*}
cd "$(dirname "$0")"
RUN="python -m torch.distributed.run --nnodes=1 --nproc-per-node=$NUM --master-addr 127.0.0.1 --master-port ${MASTER_PORT:-29577}"
echo "[1/4] profiling GEMM tile configurations on GPU $FIRST"
CUDA_VISIBLE_DEVICES=$FIRST python tune/profile_config.py --m "$M" --n "$N" --k "$K"
echo "[2/4] bandwidth curves on GPUs $DEVICES: NCCL $COMM_OP and the library's own transports"
CUDA_VISIBLE_DEVICES=$DEVICES $RUN tune/bandwidth.py --comm_op "$COMM_OP" p2p_push multimem_allreduce \
    --points "$POINTS" --reps "$REPS" --max_elements 67108864
echo "[3/4] search"
CUDA_VISIBLE_DEVICES=$DEVICES $RUN tune/search.py --m_dim "$M" --n_dim "$N" --k_dim "$K" --comm_op "$COMM_OP" --predictive_search
echo "[4/4] speed test"
CUDA_VISIBLE_DEVICES=$DEVICES $RUN test/test.py --m_dim "$M" --n_dim "$N" --k_dim "$K" --comm_op "$COMM_OP" --rmsnorm
