#!/bin/bash
# Strategy search for the bert family (CPU only).
python $(dirname $0)/../search_dist.py --num_nodes 1 --num_gpus_per_node 8 --memory_constraint 160 --mixed_precision bf16 \
    --pipeline_type pipedream_flush --default_dp_type zero2 --min_bsz 64 --max_bsz 64 --bsz_scale 1 --search_space full --sp_space tp+sp --sequence_parallel "$@"
