#!/bin/bash
set -x
set -o pipefail
export NUM_NODES=${NUM_NODES:-1}
export NUM_GPUS_PER_NODE=${NUM_GPUS_PER_NODE:-8}
export MASTER_ADDR=${MASTER_ADDR:-127.0.0.1}
export MASTER_PORT=${MASTER_PORT:-29500}
export NODE_RANK=${RANK:-0}
HERE="$(cd "$(dirname "$0")/.." && pwd)"
mkdir -p logs/profile_memory
export RUNTIME_LAUNCHER="torchrun --nnodes ${NUM_NODES} --nproc_per_node ${NUM_GPUS_PER_NODE} --master_addr ${MASTER_ADDR} --master_port ${MASTER_PORT} --node_rank ${NODE_RANK} -m hetu_galvatron_b200.cli.train_dist "
cd "$HERE" && python3 -m hetu_galvatron_b200.cli.profiler configs/profile_memory.yaml "$@" 2>&1 | tee logs/profile_memory/profile_memory.log
