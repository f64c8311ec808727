"""Hybrid-parallel training (dense and MoE models).

    torchrun --nproc-per-node 8 -m hetu_galvatron_b200.cli.train_dist configs/train_dist.yaml runtime.train.lr=1e-5

The YAML's ``runtime:`` section holds ``parallel / model / profile / train / data / ckpt / logging``; any field can
be overridden with dotted assignments.  Flags of the argparse era (``--pp_deg 2``) are translated to overrides.
Same invocation as galvatron/models/gpt/train_dist.py:76-84 and models/moe/train_dist.py:115-123 (one entry point
serves both here: the MoE path is selected by ``model.is_moe_model`` / ``num_moe_experts``).
"""
from __future__ import annotations

import sys

from ..config.loader import legacy_cli_to_overrides, load_config
from ..runtime.initialize import initialize_galvatron
from ..runtime.trainer import train


def main(argv=None):
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv:
        raise SystemExit(__doc__)
    path, rest = argv[0], argv[1:]
    overrides = legacy_cli_to_overrides(rest) if any(a.startswith("--") for a in rest) else rest
    args = load_config(path, overrides, mode="train_dist")
    initialize_galvatron(args)
    losses = train(args)
    return losses


if __name__ == "__main__":
    main()
