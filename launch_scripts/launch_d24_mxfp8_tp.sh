#!/bin/bash
# Dense depth-24 transformer (d_model 3072, 24 query / 8 KV heads, SwiGLU 8192, 8 K context) with block-scaled MXFP8
# linear layers, 2-way tensor parallelism (adjacent GPUs) x FSDP over the rest, activation checkpointing, MuonH.
# The reference trains in FP8 through TransformerEngine (`precision.py:93-99`) and has no tensor parallelism.
source "$(dirname "$0")/common.sh"
TP="${TP:-2}"
LR="${LR:-8e-3}"
TOKENS="${TOKENS:-null}"
run_pretrain "dense_d24_mxfp8_tp${TP}" --train_model transformer_gqa4 --depth 24 \
  --train_name "v2scale_mup_muonh_lr${LR}x0.1_wd0_ga_qknorm" --base_hps.eta0="$LR" --base_hps.warmup_tokens=0 \
  --base_hps.weight_decay=0 --base_hps.min_lr_mult=0.1 --max_tokens "$TOKENS" --ctx_len=8192 --micro_bsz=4 \
  --cfg.n_embd=3072 --cfg.n_head=24 --cfg.n_query_groups=8 --cfg.intermediate_size=8192 \
  --fp8=true --tp="$TP" --act_ckpt=true --use_flce=true --fsdp2=true --resume=auto --save_step=2000 --fused_comm=true
