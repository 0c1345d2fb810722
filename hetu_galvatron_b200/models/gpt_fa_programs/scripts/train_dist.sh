#!/bin/bash
# Training of the gpt_fa family on one or several nodes (set NUM_NODES / NODE_RANK / MASTER_ADDR on each node).
NUM_NODES=${NUM_NODES:-1}
NUM_GPUS_PER_NODE=${NUM_GPUS_PER_NODE:-8}
MASTER_ADDR=${MASTER_ADDR:-127.0.0.1}
MASTER_PORT=${MASTER_PORT:-29500}
NODE_RANK=${NODE_RANK:-0}
LAUNCHER="python -m torch.distributed.run --nnodes=${NUM_NODES} --nproc-per-node ${NUM_GPUS_PER_NODE} --node-rank ${NODE_RANK} --master-addr ${MASTER_ADDR} --master-port ${MASTER_PORT}"
${LAUNCHER} $(dirname $0)/../train_dist.py \
    --data-path ${DATA_PATH:?set DATA_PATH to the <prefix> of <prefix>.idx/.bin} --split 949,50,1 --global_train_batch_size 64 --train-iters 1000 --lr 1e-4 --min-lr 1e-5 --lr-decay-style cosine --lr-warmup-iters 50 \
    --adam_weight_decay 0.01 --clip-grad 1.0 --check_loss 0 --profile 0 --save-interval 500 \
    --pp_deg 1 --global_tp_deg 1 --sdp 0 --global_checkpoint 0 --vocab_tp 1 --chunks 4 \
    --pipeline_type pipedream_flush --default_dp_type zero2 --mixed_precision bf16 "$@"
