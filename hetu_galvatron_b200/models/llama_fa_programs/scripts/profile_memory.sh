#!/bin/bash
python $(dirname $0)/../profiler.py --profile_type memory --profile_mode static --profile_batch_size 8 \
    --layernum_min 1 --layernum_max 2 --max_tp_deg 8 --mixed_precision bf16 --sequence_parallel "$@"
