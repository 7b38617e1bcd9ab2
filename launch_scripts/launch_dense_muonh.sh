#!/bin/bash
# Dense GQA transformer, muP++ depth scaling, MuonH, bf16, FSDP over all GPUs (the depth-16 shape is the headline benchmark:
# d_model 2048, 16 query / 4 KV heads, head_dim 128, QK-RMSNorm, SwiGLU 5632, 8 x 4096 tokens per GPU).
# Sweeps depth and peak LR like the reference's ablation launchers (`launch_scripts/launch_phi.sh:53-90`).
source "$(dirname "$0")/common.sh"
DEPTHS="${DEPTHS:-16}"
LRS="${LRS:-1e-2}"
MICRO_BSZ="${MICRO_BSZ:-8}"
BSZ="${BSZ:-2097152}"
TOKENS="${TOKENS:-null}"
for depth in $DEPTHS; do
  for lr in $LRS; do
    act_ckpt=false; [ "$depth" -ge 20 ] && act_ckpt=true
    name="v2scale_mup_muonh_bsz${BSZ}_lr${lr}x0.1_wd0_tok${TOKENS}_ga_qknorm"
    run_pretrain "dense_d${depth}_lr${lr}" --train_model transformer_gqa4 --depth "$depth" --train_name "$name" \
      --base_hps.eta0="$lr" --base_hps.b0="$BSZ" --base_hps.warmup_tokens=0 --base_hps.weight_decay=0 \
      --base_hps.t0=10.4e9 --base_hps.min_lr_mult=0.1 --total_bsz="$BSZ" --max_tokens "$TOKENS" --micro_bsz="$MICRO_BSZ" \
      --ctx_len=4096 --use_flce=true --fsdp2=true --act_ckpt="$act_ckpt" --resume=auto --save_step=4000 \
      --cfg.intermediate_size=$((depth * 128 * 11 / 4)) --fused_comm=true
  done
done
