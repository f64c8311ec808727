#!/bin/bash
# Run scripts/train_yaml.sh and keep everything it prints in run_output.txt.
cd "$(dirname "$0")"
export PYTHONPATH="$(cd ../.. && pwd)${PYTHONPATH:+:$PYTHONPATH}"
export NPROC_PER_NODE=${NPROC_PER_NODE:-2}
exec bash scripts/train_yaml.sh "$@" 2>&1 | tee run_output.txt
