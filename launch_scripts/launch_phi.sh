#!/bin/bash
# Phi-4-mini-flash shape (SambaY 3.8 B: Mamba-1 + sliding-window attention 512 + one full-attention layer feeding the
# YOCO cross-decoder with Gated Memory Units, differential attention, vocab 200064), 8 K packed variable-length rows.
# LONG_CTX=1 reproduces the long-context recipe of the reference's README (32 K and beyond): activation checkpointing
# plus host offload of master / optimizer shards (--fsdp_save_mem).
source "$(dirname "$0")/common.sh"
CTX="${CTX:-8192}"
LR="${LR:-4e-4}"
TOKENS="${TOKENS:-1e11}"
save_mem=false; [ "${LONG_CTX:-0}" = "1" ] && save_mem=true
run_pretrain "phi4miniflash_ctx${CTX}" --train_model phi4miniflash --depth 32 \
  --train_name scaling_mup_muonh_tie_rbase_varlen --base_hps.eta0="$LR" --max_tokens "$TOKENS" --ctx_len="$CTX" \
  --micro_bsz=1 --total_bsz=$((GPUS_PER_NODE * NNODES * CTX * 8)) --use_flce=true --fsdp2=true --act_ckpt=true \
  --fsdp_save_mem="$save_mem" --resume=auto --save_step=1000 --fused_comm=true
