#!/bin/bash
# Measures all-reduce / p2p bandwidth, all-reduce and all-to-all latency tables, the compute/communication overlap
# coefficient and this package's own NVLink kernels on one node, and writes ../hardware_configs/*.json.
NUM_GPUS_PER_NODE=${NUM_GPUS_PER_NODE:-8}
python -m torch.distributed.run --nnodes=1 --nproc-per-node ${NUM_GPUS_PER_NODE} --master-addr 127.0.0.1 --master-port ${MASTER_PORT:-29500} \
    -m hetu_galvatron_b200.profiler.hardware_profiler --num_nodes 1 --num_gpus_per_node ${NUM_GPUS_PER_NODE} "$@"
