#!/bin/bash
# Measures the slow-down of a GEMM and an all-reduce running together and writes ../hardware_configs/overlap_coefficient.json.
NUM_GPUS_PER_NODE=${NUM_GPUS_PER_NODE:-8}
python -m torch.distributed.run --nnodes=1 --nproc-per-node ${NUM_GPUS_PER_NODE} --master-addr 127.0.0.1 --master-port ${MASTER_PORT:-29500} \
    $(dirname $0)/../profile_overlap.py --num_nodes 1 --num_gpus_per_node ${NUM_GPUS_PER_NODE} "$@"
