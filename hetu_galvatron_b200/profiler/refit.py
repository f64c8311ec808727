"""Re-fit of the cost model's backward / forward ratio to this hardware and these kernels.

The cost model takes the backward pass as a fixed multiple of the profiled forward time (2 in the reference,
galvatron/core/cost_model/components/layer_cost.py:72-80).  With hand-written kernels the multiple is a property of
the kernels (the flash-attention backward costs about five forwards, the GEMMs exactly two), so it is measured:

    python -m hetu_galvatron_b200.profiler.refit configs/profile_computation_b200.yaml

launches the training entry point (``$RUNTIME_LAUNCHER``) for the minimum and maximum layer count of the YAML with the
full iteration timed (forward + backward + optimizer), reads the forward-only numbers the computation profile left
in ``configs/computation_profiling_*.json`` and writes

    hardware_configs/b200_refit.json   {"backward_forward_ratio": r, ...}

where ``1 + r = (T_full(Lmax) - T_full(Lmin)) / (T_fwd(Lmax) - T_fwd(Lmin))``.  The search engine picks the file up
from the hardware-profile directory.
"""
from __future__ import annotations

import json
import os
import sys
from typing import Dict, Optional

from ..config.loader import load_config
from ..config.model_config import model_name, resolve_model_config
from ..utils.config_utils import read_json_config, write_json_config
from .model import ModelProfiler


def ratio_from_times(fwd: Dict[str, float], full: Dict[str, float], lmin: int, lmax: int, bsz: int, seq: int) -> float:
    k = lambda L: "layernum%d_bsz%d_seq%d" % (L, bsz, seq)  # noqa: E731
    d_fwd = fwd[k(lmax)] - fwd[k(lmin)]
    d_full = full[k(lmax)] - full[k(lmin)]
    if d_fwd <= 0 or d_full <= d_fwd:
        raise ValueError("inconsistent timings: forward %s, full %s" % (d_fwd, d_full))
    return d_full / d_fwd - 1.0


def main(argv=None, run=os.system, out_dir: Optional[str] = None):
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv:
        raise SystemExit(__doc__)
    args = load_config(argv[0], argv[1:], mode="model_profiler")
    resolve_model_config(args)
    prof = ModelProfiler(args)
    work = os.environ.get("HG_PROFILE_DIR") or os.getcwd()
    prof.set_profiler_launcher(work, model_name(args))
    if args.profile_type != "computation" or args.profile_mode != "static":
        raise SystemExit("the refit uses a static computation profile")
    bsz = prof.get_global_batch_size_list()[0]
    seq = prof.get_seq_length_tuple_list()[0][0]
    lmin, lmax = args.profile_layernum_min, args.profile_layernum_max
    base = dict(prof.get_basic_overrides_dict())
    base.update({"runtime.profile.profile_forward": 0, "runtime.profile.save_profiled_iteration_time": 1,
                 "runtime.train.global_batch_size": bsz, "runtime.train.seq_length": seq})
    log_dir = os.path.join(work, "logs/profile_refit")
    os.makedirs(log_dir, exist_ok=True)
    for L in (lmin, lmax):
        ov = dict(base)
        ov["runtime.model.num_layers"] = L
        run(prof._command(ov, log_dir, "full_layernum_%d" % L))
    fwd = read_json_config(prof.time_profiling_path())
    full = read_json_config(prof._config_path("iteration"))
    r = ratio_from_times(fwd, full, lmin, lmax, bsz, seq)
    out_dir = out_dir or os.path.join(work, "hardware_configs")
    path = os.path.join(out_dir, "b200_refit.json")
    cfg = read_json_config(path) if os.path.exists(path) else {}
    cfg.update({"backward_forward_ratio": r, "measured_with": {"model": model_name(args), "bsz": bsz, "seq": seq,
                                                                "layers": [lmin, lmax]}})
    write_json_config(cfg, path)
    print("backward / forward ratio %.4f written to %s" % (r, path))
    return r


if __name__ == "__main__":
    main()
