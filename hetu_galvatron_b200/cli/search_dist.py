"""Parallelism-strategy search.

    python -m hetu_galvatron_b200.cli.search_dist configs/search_dist.yaml search_engine.hardware_info.memory_constraint=80

Reads the profiled computation / memory / hardware JSON files named in the ``search_engine:`` section, runs the
dynamic-programming search over per-layer strategies for every candidate batch size and writes
``galvatron_config_<model>_<N>nodes_<G>gpus_per_node_<M>GB_<precision>[_bsz..].json``.
Same invocation and outputs as galvatron/models/gpt/search_dist.py:11-33.
"""
from __future__ import annotations

import os
import sys

from ..config.loader import load_config
from ..config.model_config import model_layer_configs, model_name, resolve_model_config
from ..search.engine import GalvatronSearchEngine


def main(argv=None):
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv:
        raise SystemExit(__doc__)
    args = load_config(argv[0], argv[1:], mode="search")
    resolve_model_config(args)
    engine = GalvatronSearchEngine(args)
    # profiled JSON files are read from <dir>/configs/ and the result is written there (the directory the profilers
    # were run from: HG_PROFILE_DIR, else the current directory)
    work_dir = os.environ.get("HG_PROFILE_DIR") or os.getcwd()
    engine.set_search_engine_info(work_dir, model_layer_configs(args), model_name(args))
    engine.initialize_search_engine()
    return engine.parallelism_optimization()


if __name__ == "__main__":
    main()
