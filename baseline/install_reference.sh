#!/bin/bash
# Installs the unmodified reference into baseline/_ref (git-ignored) for `bench.py --impl reference`.
#   usage: baseline/install_reference.sh <path to the reference checkout>
# Steps: (1) copy the checkout to a scratch directory (its setup.py writes into the tree); (2) put helpers.cpp and
# Makefile where setup.py's data_files expects them (it names galvatron/site_package/megatron/core/datasets/, the
# files live in galvatron/core/runtime/datasets/megatron/); (3) pip install offline, without dependency resolution;
# (4) copy the data files that setup.py does not package but the reference reads at run time, byte for byte:
# the YAML configurations, the launcher scripts, and the dataset helper's Makefile + helpers.cpp (the reference runs
# `make -C` in its installed datasets directory at start-up).  No Python source of the reference is touched.
set -euo pipefail
SRC=${1:?path to the reference checkout}
HERE=$(cd "$(dirname "$0")" && pwd)
TMP=$(mktemp -d /tmp/hg_ref_install.XXXXXX)
cp -r "$SRC" "$TMP/src"
mkdir -p "$TMP/src/galvatron/site_package/megatron/core/datasets"
cp "$TMP/src/galvatron/core/runtime/datasets/megatron/helpers.cpp" "$TMP/src/galvatron/core/runtime/datasets/megatron/Makefile" \
   "$TMP/src/galvatron/site_package/megatron/core/datasets/"
# A fresh target and no --upgrade: setup.py's data_files land in a second top-level "galvatron" directory, and with
# --upgrade pip replaces the package directory by that one (the Python files vanish); without it pip keeps the package.
if [ -d "$HERE/_ref" ]; then mv "$HERE/_ref" "$TMP/old_ref"; fi
python -m pip install --no-index --no-build-isolation --no-deps --find-links /opt/wheelhouse \
   --target "$HERE/_ref" "$TMP/src"
(cd "$SRC" && find galvatron \( -name '*.yaml' -o -name '*.sh' -o -name 'Makefile' -o -name 'helpers.cpp' \) -print0 \
   | while IFS= read -r -d '' f; do mkdir -p "$HERE/_ref/$(dirname "$f")"; cp "$f" "$HERE/_ref/$f"; done)
echo "installed into $HERE/_ref"
