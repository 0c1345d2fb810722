#!/bin/bash
# Synthetic-data training of the llama_fa family on one 8-GPU node.
NUM_GPUS_PER_NODE=${NUM_GPUS_PER_NODE:-8}
python -m torch.distributed.run --nnodes=1 --nproc-per-node ${NUM_GPUS_PER_NODE} --master-addr 127.0.0.1 --master-port ${MASTER_PORT:-29500} \
    $(dirname $0)/../train_dist_random.py \
    --global_train_batch_size 16 --train-iters 25 --lr 1e-4 --adam_weight_decay 0.01 --check_loss 0 --profile 1 \
    --pp_deg 1 --global_tp_deg 1 --sdp 0 --global_checkpoint 0 --vocab_tp 1 --chunks 1 \
    --pipeline_type pipedream_flush --default_dp_type zero2 --mixed_precision bf16 "$@"
