"""``bench.py --impl reference``: the unmodified reference, installed into ``baseline/_ref``, through its own
entry point (``galvatron.models.gpt.train_dist``) -- or one JSON line saying why that cannot run here.

The reference's import chain needs, besides torch and flash-attn's attention kernels:

* ``hydra`` and ``omegaconf`` (``galvatron/core/arguments.py`` composes every configuration through Hydra),
* ``dropout_layer_norm``, the CUDA extension built from flash-attention's ``csrc/layer_norm`` (imported by
  ``flash_attn.ops.rms_norm`` which ``galvatron/core/runtime/transformer/norm.py:3`` imports at module load).

The probe below imports exactly those; whatever is missing is named in the ``unavailable`` line.  Nothing of this
repository's models, kernels or engine is put on the reference's path, and no stand-in for a missing dependency is
provided (a stand-in for the layer-norm extension would be one of this repository's kernels on that path).
"""
from __future__ import annotations

import importlib
import json
import os
import sys

REF_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref")
NEEDS = ("hydra", "omegaconf", "dropout_layer_norm", "flash_attn")


def probe():
    """Names of what stops the reference from importing on this image ([] when it imports)."""
    if not os.path.isdir(os.path.join(REF_DIR, "galvatron")):
        return ["baseline/_ref (the reference is not installed)"]
    missing = []
    for name in NEEDS:
        try:
            importlib.import_module(name)
        except Exception as e:  # ImportError, or a binary built against another torch
            missing.append("%s (%s)" % (name, type(e).__name__))
    if missing:
        return missing
    sys.path.insert(0, REF_DIR)
    try:
        importlib.import_module("galvatron.core.runtime.models.builder")
        importlib.import_module("galvatron.core.arguments")
    except Exception as e:
        return ["galvatron import: %s: %s" % (type(e).__name__, str(e)[:160])]
    return []


def run(a):
    rank = int(os.environ.get("RANK", "0"))
    missing = probe()
    if not missing:
        # All dependencies present (not the case on the image this was written on): the reference's stock path is
        # its launcher script with a YAML; running it from here has never been possible to validate, so say so
        # rather than print a number from an untested harness.
        missing = ["a validated launcher: the reference imports on this image but its run was never exercised"]
    if rank == 0:
        print(json.dumps({"impl": "reference", "unavailable":
                          "reference installed into baseline/_ref but cannot run: missing " + ", ".join(missing)}))
    return 0
