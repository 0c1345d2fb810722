#!/bin/bash
python $(dirname $0)/../profiler.py --profile_type computation --profile_mode static --profile_batch_size 1 \
    --layernum_min 1 --layernum_max 2 --mixed_precision bf16 "$@"
