#!/bin/bash
# HuggingFace checkpoint of a T5 model -> one file per block, loadable by --load (with --initialize_on_meta 1) into a model
# built with --relative_attention_num_buckets 32 --t5_feed_forward relu.
#   bash convert_t5_h2g.sh <huggingface checkpoint dir> <output dir>
python -m hetu_galvatron_b200.tools.checkpoint_convert_h2g --model_type t5 --input_checkpoint "$1" --output_dir "$2"
