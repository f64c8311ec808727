#!/bin/bash
# Distributed checkpoint -> HuggingFace names.  Usage: convert_llama_g2h.sh <ckpt dir> <iteration> <output dir> [model config]
python3 -m hetu_galvatron_b200.cli.checkpoint_convert_g2h --model_type llama --input_checkpoint "$1" --load_iteration "$2" \
    --output_dir "$3" --model_config "${4:-llama2-7b}"
