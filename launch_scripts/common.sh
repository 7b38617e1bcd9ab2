#!/bin/bash
# Shared settings of the launch scripts: one process per GPU under torchrun, NCCL over NVLink / NVSwitch for the
# torch.distributed plumbing, the package's peer-memory kernels for the hot collectives (--fused_comm).
# Environment knobs: NNODES, NODE_RANK, GPUS_PER_NODE, MASTER_ADDR (host:port), DATA_DIR, VAL_DIR, OUT_DIR, LOGDIR,
# WANDB_PROJECT (unset = no wandb).  DATA_DIR=synthetic trains on uniform-random tokens.
set -euo pipefail
REPO="$(cd "$(dirname "${BASH_SOURCE[0]}")/.." && pwd)"
export NCCL_DEBUG="${NCCL_DEBUG:-WARN}"
export NCCL_NVLS_ENABLE="${NCCL_NVLS_ENABLE:-1}"          # in-switch reductions for the NCCL collectives that remain
export NCCL_CUMEM_ENABLE="${NCCL_CUMEM_ENABLE:-1}"
export PYTORCH_CUDA_ALLOC_CONF="${PYTORCH_CUDA_ALLOC_CONF:-expandable_segments:True}"
NNODES="${NNODES:-1}"
NODE_RANK="${NODE_RANK:-0}"
GPUS_PER_NODE="${GPUS_PER_NODE:-8}"
MASTER_ADDR="${MASTER_ADDR:-127.0.0.1:29500}"
DATA_DIR="${DATA_DIR:-synthetic}"
VAL_DIR="${VAL_DIR:-}"
OUT_DIR="${OUT_DIR:-$REPO/out}"
LOGDIR="${LOGDIR:-$OUT_DIR/logs}"
mkdir -p "$LOGDIR"
[ -f "$REPO/archscale_b200/_C.so" ] || python -m archscale_b200.build

# run_pretrain <run name> <pretrain.py flags...>
run_pretrain() {
  local run_name="$1"; shift
  local extra=()
  [ -n "$VAL_DIR" ] && extra+=(--val_data_dir "$VAL_DIR")
  [ -n "${WANDB_PROJECT:-}" ] && extra+=(--wandb_project "$WANDB_PROJECT")
  echo "== $run_name: $NNODES node(s) x $GPUS_PER_NODE GPU(s), rendezvous $MASTER_ADDR"
  LIGHTNING_ARTIFACTS_DIR="$OUT_DIR/$run_name" python -m torch.distributed.run --nnodes="$NNODES" \
    --nproc-per-node="$GPUS_PER_NODE" --node-rank="$NODE_RANK" --rdzv-backend=c10d --rdzv-endpoint="$MASTER_ADDR" \
    "$REPO/pretrain.py" --train_data_dir "$DATA_DIR" "${extra[@]}" "$@" 2>&1 | tee -a "$LOGDIR/train_${run_name}_${HOSTNAME:-node}.log"
}
