#!/bin/bash
set -x
set -o pipefail
HERE="$(cd "$(dirname "$0")/.." && pwd)"
mkdir -p logs/search_engine
cd "$HERE" && python3 -m hetu_galvatron_b200.cli.search_dist "${1:-$HERE/configs/search_dist.yaml}" "${@:2}" 2>&1 | tee logs/search_engine/search_engine.log
