#!/bin/bash
# Plumbing check without a GPU: two gloo ranks, fp32, a 2-layer dense GQA transformer on synthetic tokens for a few
# optimizer steps, checkpoint at the end (role of the reference's `launch_scripts/launch_test.sh`).
export GPUS_PER_NODE="${GPUS_PER_NODE:-2}"
source "$(dirname "$0")/common.sh"
CUDA_VISIBLE_DEVICES="" run_pretrain "plumbing_cpu" --train_model transformer_gqa4 --depth 8 --train_name scaling_mup_muon \
  --precision fp32 --ctx_len=512 --micro_bsz=2 --total_bsz=2048 --max_tokens 20480 --use_flce=true --fsdp2=true \
  --cfg.n_layer=2 --cfg.n_embd=256 --cfg.n_head=2 --cfg.n_query_groups=1 --cfg.intermediate_size=1024 --cfg.ar=none
