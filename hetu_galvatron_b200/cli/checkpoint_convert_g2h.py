"""Distributed checkpoint of this framework -> HuggingFace parameter names (one ``pytorch_model.bin`` + config).

    python -m hetu_galvatron_b200.cli.checkpoint_convert_g2h --load_iteration 1000 --input_checkpoint <ckpt dir> \\
        --output_dir <dir> --model_config llama2-7b --model_type llama

Tensor-parallel shards are merged (QKV un-interleaved from the grouped-query layout, gate/up split, vocabulary
padding removed).  Same tool as galvatron/tools/checkpoint_convert_g2h.py:1-271.
"""
from __future__ import annotations

import argparse
import json
import os

import torch

from ..config.model_config import create_hf_config, resolve_model_config
from ..config.schema import GalvatronRuntimeArgs
from ..models.spec import spec_from_args
from ..runtime.checkpoint import export_to_hf


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--load_iteration", type=int, required=True)
    ap.add_argument("--input_checkpoint", required=True)
    ap.add_argument("--output_dir", required=True)
    ap.add_argument("--model_config", required=True, help="model YAML path or zoo name")
    ap.add_argument("--model_type", required=True)
    ap.add_argument("--seq_length", type=int, default=4096)
    a = ap.parse_args(argv)
    args = GalvatronRuntimeArgs(model=dict(model_config_path=a.model_config), train=dict(seq_length=a.seq_length, global_batch_size=1))
    resolve_model_config(args)
    spec = spec_from_args(args)
    sd = export_to_hf(a.input_checkpoint, a.load_iteration, spec)
    os.makedirs(a.output_dir, exist_ok=True)
    torch.save(sd, os.path.join(a.output_dir, "pytorch_model.bin"))
    try:
        cfg = create_hf_config(args)
        with open(os.path.join(a.output_dir, "config.json"), "w") as f:
            json.dump(cfg.to_dict(), f, indent=2, default=str)
    except Exception as e:  # the HF config class of an unusual architecture may be unavailable
        print("config.json not written: %s" % e)
    print("wrote %d tensors to %s" % (len(sd), a.output_dir))
    return sd


if __name__ == "__main__":
    main()
