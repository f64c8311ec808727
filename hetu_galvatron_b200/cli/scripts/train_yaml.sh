#!/bin/bash
# Launch hybrid-parallel training: scripts/train_yaml.sh [config.yaml] [runtime.section.key=value ...]
set -x
set -o pipefail
export PYTORCH_CUDA_ALLOC_CONF="expandable_segments:True"
export NCCL_DEBUG=${NCCL_DEBUG:-WARN}

NNODES=${NNODES:=1}
NPROC_PER_NODE=${NPROC_PER_NODE:=8}
NODE_RANK=${NODE_RANK:=0}
MASTER_ADDR=${MASTER_ADDR:=127.0.0.1}
MASTER_PORT=${MASTER_PORT:=12345}
HERE="$(cd "$(dirname "$0")/.." && pwd)"

CONFIG="$HERE/configs/train_dist.yaml"
if [[ "$1" == *.yaml ]]; then CONFIG="$1"; shift; fi
mkdir -p logs/runtime
torchrun --nnodes=$NNODES --nproc-per-node=$NPROC_PER_NODE --node-rank=$NODE_RANK \
  --master-addr=$MASTER_ADDR --master-port=$MASTER_PORT \
  -m hetu_galvatron_b200.cli.train_dist "$CONFIG" "$@" 2>&1 | tee logs/runtime/train_runtime.log
