#!/bin/bash
set -x
set -o pipefail
export NUM_NODES=${NUM_NODES:-1}
export NUM_GPUS_PER_NODE=${NUM_GPUS_PER_NODE:-8}
export MASTER_ADDR=${MASTER_ADDR:-127.0.0.1}
export MASTER_PORT=${MASTER_PORT:-29500}
export NODE_RANK=${RANK:-0}
HERE="$(cd "$(dirname "$0")/.." && pwd)"
mkdir -p logs/profile_hardware
cd "$HERE" && python3 -m hetu_galvatron_b200.cli.profile_hardware configs/profile_hardware.yaml "$@" 2>&1 | tee logs/profile_hardware/profile_hardware.log
for s in profile_allreduce profile_p2p profile_allreduce_sp profile_all2all_sp; do sh scripts/$s.sh; done
