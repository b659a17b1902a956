#!/bin/bash
# A Megatron-style launch script: the tuner reads the --flag value pairs (shell variables defined
# as NAME=value above their use are substituted).
LAYERS=24
HIDDEN=4096
EXPERTS=32

python pretrain_gpt.py \
    --num-layers ${LAYERS} \
    --hidden-size ${HIDDEN} \
    --ffn-hidden-size 11008 \
    --num-attention-heads 32 \
    --num-query-groups 8 \
    --vocab-size 128256 \
    --seq-length 4096 \
    --num-experts ${EXPERTS} \
    --moe-ffn-hidden-size 2048 \
    --moe-router-topk 4 \
    --first-k-dense-replace 2 \
    --global-batch-size 64
