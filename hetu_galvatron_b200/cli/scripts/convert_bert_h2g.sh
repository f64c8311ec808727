#!/bin/bash
# HuggingFace BERT (masked-LM) checkpoint -> one file per module (key regrouping only).
INPUT_PATH=${1:-/path/to/huggingface/bert/checkpoint/}
OUTPUT_PATH=${2:-/path/to/split/bert/checkpoint/}
python3 -m hetu_galvatron_b200.cli.checkpoint_convert_h2g --model_type bert-mlm \
    --input_checkpoint "$INPUT_PATH" --output_dir "$OUTPUT_PATH"
