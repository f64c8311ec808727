"""Model profiling: plan and launch the profiling runs, then post-process their measurements.

    RUNTIME_LAUNCHER="torchrun --nnodes 1 --nproc_per_node 1 -m hetu_galvatron_b200.cli.train_dist" \\
        python -m hetu_galvatron_b200.cli.profiler configs/profile_computation.yaml

``profile_flow_control``: ``all`` (launch + process), ``scripts_only`` (write the command list to
``scripts/<type>_profile_scripts_<unit>.sh``), ``launch_only``, ``data_only`` (process existing raw JSON).
Same invocation as galvatron/models/gpt/profiler.py:7-22.
"""
from __future__ import annotations

import os
import sys

from ..config.loader import load_config
from ..config.model_config import model_name, resolve_model_config
from ..profiler.model import ModelProfiler


def main(argv=None):
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv:
        raise SystemExit(__doc__)
    args = load_config(argv[0], argv[1:], mode="model_profiler")
    resolve_model_config(args)
    prof = ModelProfiler(args)
    work_dir = os.environ.get("HG_PROFILE_DIR") or os.getcwd()
    prof.set_profiler_launcher(work_dir, model_name(args))
    prof.launch_profiling_scripts()
    prof.process_profiled_data()
    return prof


if __name__ == "__main__":
    main()
