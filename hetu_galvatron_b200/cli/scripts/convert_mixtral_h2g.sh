#!/bin/bash
# HuggingFace checkpoint -> per-module split files.  Usage: convert_mixtral_h2g.sh <hf checkpoint dir> <output dir>
python3 -m hetu_galvatron_b200.cli.checkpoint_convert_h2g --model_type mixtral --input_checkpoint "$1" --output_dir "$2"
