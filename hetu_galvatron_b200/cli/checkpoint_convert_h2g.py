"""HuggingFace checkpoint -> per-module split files that the runtime loads under any parallel strategy.

    python -m hetu_galvatron_b200.cli.checkpoint_convert_h2g --model_type llama --input_checkpoint <hf dir> --output_dir <dir>

``model_type``: ``llama`` (also qwen / mistral dense), ``gpt``, ``mixtral``, ``bert-mlm`` (key regrouping only, as in the
reference: no BERT model is built from it).  Output layout: one ``.pt`` per module
(``model_embed_tokens.pt``, ``model_layers_{i}.pt``, ``model_norm.pt``, ``lm_head.pt``) with the HF key names minus the
module prefix.  Same tool as galvatron/tools/checkpoint_convert_h2g.py:140-159.
"""
from __future__ import annotations

import argparse

from ..runtime.checkpoint import convert_hf_to_split, read_hf_checkpoint


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--model_type", required=True, choices=["llama", "gpt", "mixtral", "qwen", "mistral", "bert-mlm"])
    ap.add_argument("--input_checkpoint", required=True)
    ap.add_argument("--output_dir", required=True)
    a = ap.parse_args(argv)
    sd = read_hf_checkpoint(a.input_checkpoint)
    files = convert_hf_to_split(sd, a.model_type, a.output_dir)
    print("wrote %d files to %s" % (len(files), a.output_dir))
    return files


if __name__ == "__main__":
    main()
