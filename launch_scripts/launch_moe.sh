#!/bin/bash
# Fine-grained MoE (transformer_gqa4_h2_moe: 64 routed SwiGLU experts + 1 shared, token-choice top-8, SqrtGate, global
# auxiliary load-balance loss), FSDP for the dense part, expert parallelism over the GPUs of a node.
# Flags follow the reference's MoE launcher (`launch_scripts/launch_moe.sh:56-98`); --ep / --fused_comm are additions.
source "$(dirname "$0")/common.sh"
DEPTHS="${DEPTHS:-8}"
LRS="${LRS:-8e-3}"
SPARSITY="${SPARSITY:-8}"
TOPK="${TOPK:-8}"
EP="${EP:-$GPUS_PER_NODE}"
BSZ="${BSZ:-4194304}"
TOKENS="${TOKENS:-10.4e9}"
AUX_GAMMA="${AUX_GAMMA:-1e-2}"
for depth in $DEPTHS; do
  for lr in $LRS; do
    micro_bsz=16; [ "$depth" -ge 24 ] && micro_bsz=8
    act_ckpt=false; [ "$depth" -ge 20 ] && act_ckpt=true
    name="v2scale_mup_muonh_bsz${BSZ}_lr${lr}x0.1_wd0_tok${TOKENS}_gblaux${AUX_GAMMA}_ga_qknorm_sgate_shexp"
    run_pretrain "moe_d${depth}_s${SPARSITY}_k${TOPK}_lr${lr}" --train_model transformer_gqa4_h2_moe --depth "$depth" \
      --sparsity="$SPARSITY" --top_k="$TOPK" --share_expert=true --global_aux=true --sqrt_gate=true \
      --aux_style=switch --aux_gamma="$AUX_GAMMA" --train_name "$name" \
      --base_hps.eta0="$lr" --base_hps.b0="$BSZ" --base_hps.warmup_tokens=0 --base_hps.weight_decay=0 \
      --base_hps.t0=10.4e9 --base_hps.min_lr_mult=0.1 --total_bsz="$BSZ" --max_tokens "$TOKENS" --micro_bsz="$micro_bsz" \
      --ctx_len=4096 --use_flce=true --fsdp2=true --act_ckpt="$act_ckpt" --resume=auto --save_step=4000 \
      --ep="$EP" --fused_comm=true
  done
done
