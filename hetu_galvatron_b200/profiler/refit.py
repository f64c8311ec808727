"""Re-fit of the cost model's backward / forward ratio to this hardware and these kernels.

The cost model takes the backward pass as a fixed multiple of the profiled forward time (2 in the reference,
galvatron/core/cost_model/components/layer_cost.py:72-80).  With hand-written kernels the multiple is a property of
the kernels (the flash-attention backward costs about five forwards, the GEMMs exactly two), so it is measured:

    python -m hetu_galvatron_b200.profiler.refit configs/profile_computation_b200.yaml

launches the training entry point (``$RUNTIME_LAUNCHER``) for the minimum and maximum layer count of the YAML with the
full iteration timed (forward + backward + optimizer), reads the forward-only numbers the computation profile left
in ``configs/computation_profiling_*.json`` and writes

    hardware_configs/b200_refit.json   {"backward_forward_ratio": r, ...}

where ``1 + r = (T_full(Lmax) - T_full(Lmin) - o * dL) / (T_fwd(Lmax) - T_fwd(Lmin))`` and ``o`` is the part of a layer's
iteration that does not scale with the number of micro-batches (AdamW, gradient norm, gradient-buffer handling), kept
as its own term (``optimizer_ms_per_layer``).  ``o`` is measured, not derived: the same two layer counts are run a
second time with two micro-batches per step (twice the batch, ``chunks=2``); with ``d1`` / ``d2`` the per-layer
iteration times at one / two micro-batches, ``x = d2 - d1`` is a micro-batch's forward + backward and ``o = 2 d1 - d2``.
(Streaming 34 bytes per parameter at the copy bandwidth, the analytic estimate used when the second pair of runs is
missing, gives 0.98 ms for a Llama-2-7B layer; the measurement is about twice that.)  The search engine picks the file
up from the hardware-profile directory.
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


def optimizer_ms_per_layer(parameter_size_mb: float, hbm_gbs: float) -> float:
    """``parameter_size_mb`` is the memory profile's figure (model-state MB / 4).  Bytes streamed per step: read
    fp32 gradient, master, two moments, write master, two moments (28) + bf16 parameter (2) + gradient-norm read (4)."""
    state_mb = 4.0 * parameter_size_mb
    return state_mb * (34.0 / 18.0) / 1024.0 / hbm_gbs * 1e3


def ratio_from_times(fwd: Dict[str, float], full: Dict[str, float], lmin: int, lmax: int, bsz: int, seq: int,
                     optimizer_ms: float = 0.0) -> float:
    k = lambda L: "layernum%d_bsz%d_seq%d" % (L, bsz, seq)  # noqa: E731
    d_fwd = fwd[k(lmax)] - fwd[k(lmin)]
    d_full = full[k(lmax)] - full[k(lmin)] - optimizer_ms * (lmax - lmin)
    if d_fwd <= 0 or d_full <= d_fwd:
        raise ValueError("inconsistent timings: forward %s, full %s" % (d_fwd, d_full))
    return d_full / d_fwd - 1.0


def optimizer_ms_from_accumulation(full: Dict[str, float], lmin: int, lmax: int, bsz: int, seq: int) -> Optional[float]:
    """Per-layer time that does not scale with the micro-batch count, from iteration times at one micro-batch
    (batch ``bsz``) and two (batch ``2*bsz``): ``o = 2 * d1 - d2`` with ``d`` the per-layer differences.  ``None`` when
    the two-micro-batch runs are missing or the result is not positive."""
    k = lambda L, b: "layernum%d_bsz%d_seq%d" % (L, b, seq)  # noqa: E731
    try:
        d1 = (full[k(lmax, bsz)] - full[k(lmin, bsz)]) / (lmax - lmin)
        d2 = (full[k(lmax, 2 * bsz)] - full[k(lmin, 2 * bsz)]) / (lmax - lmin)
    except KeyError:
        return None
    o = 2.0 * d1 - d2
    return o if 0.0 < o < d1 else None


def measured_hbm_gbs(default: float = 6500.0) -> float:
    here = os.path.dirname(os.path.abspath(__file__))
    for up in (os.path.join(here, "..", ".."), os.getcwd()):
        p = os.path.join(up, "MEASURED_PEAKS.json")
        if os.path.exists(p):
            return float(json.load(open(p)).get("hbm_gbs", default))
    return default


def main(argv=None, run=os.system, out_dir: Optional[str] = None, no_launch: bool = False):
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
    # The per-step (optimizer) term is a small difference of iteration times, so it is taken over a longer lever than
    # the ratio: lmin against four times lmax layers (HG_REFIT_ACC_LAYERS overrides), one and two micro-batches.
    lacc = int(os.environ.get("HG_REFIT_ACC_LAYERS", 4 * lmax))
    if not no_launch:
        for L in sorted({lmin, lmax, lacc}):
            ov = dict(base)
            ov["runtime.model.num_layers"] = L
            run(prof._command(ov, log_dir, "full_layernum_%d" % L))
        for L in sorted({lmin, lacc}):     # the same with two micro-batches per step: separates the per-step part
            ov = dict(base)
            ov.update({"runtime.model.num_layers": L, "runtime.train.global_batch_size": 2 * bsz, "runtime.train.chunks": 2})
            run(prof._command(ov, log_dir, "full_layernum_%d_chunks2" % L))
    fwd = read_json_config(prof.time_profiling_path())
    full = read_json_config(prof._config_path("iteration"))
    opt_ms = 0.0
    mem_path = prof.memory_profiling_path()
    if os.path.exists(mem_path):
        mem = read_json_config(mem_path)
        for key in ("layertype_0_sp", "layertype_0"):
            if key in mem and str(seq) in mem[key]:
                opt_ms = optimizer_ms_per_layer(mem[key][str(seq)]["parameter_size"], measured_hbm_gbs())
                break
    measured = optimizer_ms_from_accumulation(full, lmin, lacc, bsz, seq)
    if measured is None:
        measured = optimizer_ms_from_accumulation(full, lmin, lmax, bsz, seq)
    if measured is not None:
        opt_ms = measured
    r = ratio_from_times(fwd, full, lmin, lmax, bsz, seq, opt_ms)
    out_dir = out_dir or os.path.join(work, "hardware_configs")
    path = os.path.join(out_dir, "b200_refit.json")
    cfg = read_json_config(path) if os.path.exists(path) else {}
    cfg.update({"backward_forward_ratio": r, "optimizer_ms_per_layer": opt_ms, "measured_with": {"model": model_name(args), "bsz": bsz, "seq": seq,
                                                                "layers": [lmin, lmax],
                                                                "optimizer_term_layers": [lmin, lacc]}})
    write_json_config(cfg, path)
    print("backward / forward ratio %.4f written to %s" % (r, path))
    return r


if __name__ == "__main__":
    main()
