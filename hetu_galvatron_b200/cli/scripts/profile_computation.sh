#!/bin/bash
set -x
set -o pipefail
HERE="$(cd "$(dirname "$0")/.." && pwd)"
mkdir -p logs/profile_computation
export RUNTIME_LAUNCHER="torchrun --nnodes 1 --nproc_per_node 1 --master_addr 127.0.0.1 -m hetu_galvatron_b200.cli.train_dist "
cd "$HERE" && python3 -m hetu_galvatron_b200.cli.profiler configs/profile_computation.yaml "$@" 2>&1 | tee logs/profile_computation/profile_computation.log
