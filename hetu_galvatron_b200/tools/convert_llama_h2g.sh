#!/bin/bash
# HuggingFace checkpoint of a llama model -> one file per block, loadable by --load with --initialize_on_meta 1.
#   bash convert_llama_h2g.sh <huggingface checkpoint dir> <output dir>
python -m hetu_galvatron_b200.tools.checkpoint_convert_h2g --model_type llama --input_checkpoint "$1" --output_dir "$2"
