"""Hardware profiling: write the sweep scripts and measure the compute / communication overlap coefficient.

    python -m hetu_galvatron_b200.cli.profile_hardware configs/profile_hardware.yaml
    sh scripts/profile_allreduce.sh; sh scripts/profile_p2p.sh; sh scripts/profile_allreduce_sp.sh; sh scripts/profile_all2all_sp.sh

The scripts run ``hetu_galvatron_b200.profiler.hardware`` under torchrun and fill ``hardware_configs/*.json``.
Same flow as galvatron/profile_hardware/profile_hardware.py:7-21.
"""
from __future__ import annotations

import os
import sys

from ..config.loader import load_config
from ..profiler.hardware import HardwareProfiler


def main(argv=None, run_overlap: bool = True):
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv:
        raise SystemExit(__doc__)
    args = load_config(argv[0], argv[1:], mode="profiler_hardware")
    prof = HardwareProfiler(args)
    prof.set_path(os.environ.get("HG_PROFILE_DIR") or os.getcwd())
    prof.profile_bandwidth()
    prof.profile_sp_bandwidth()
    if run_overlap and os.environ.get("HG_SKIP_OVERLAP", "0") != "1":
        prof.profile_overlap()
    return prof


if __name__ == "__main__":
    main()
