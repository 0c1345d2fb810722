#!/bin/bash
# Distributed checkpoint of a t5 run with the relative position bias (iter_N/<block>/<tp rank>.pt) -> HuggingFace state dict
# + config.json. Defined while the bias tables of a stack agree (HuggingFace keeps one per stack).
#   bash convert_t5_g2h.sh <checkpoint dir> <output dir> <iteration> [meta config json]
META=${4:-$(dirname $0)/../models/meta_configs/t5-large.json}
python -m hetu_galvatron_b200.tools.checkpoint_convert_g2h --model_type t5 --input_checkpoint "$1" --output_dir "$2" \
    --load_iteration "$3" --model_config "$META"
