#!/bin/bash
# Distributed checkpoint of a llama run (iter_N/<block>/<tp rank>.pt) -> HuggingFace state dict + config.json.
#   bash convert_llama_g2h.sh <checkpoint dir> <output dir> <iteration> [meta config json]
META=${4:-$(dirname $0)/../models/meta_configs/llama-7b.json}
python -m hetu_galvatron_b200.tools.checkpoint_convert_g2h --model_type llama --input_checkpoint "$1" --output_dir "$2" \
    --load_iteration "$3" --model_config "$META"
