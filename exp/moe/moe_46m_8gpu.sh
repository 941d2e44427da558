#!/bin/bash
# Token-dropping MoE, 46m backbone, 8 GPUs, fp16
# Counterpart of the reference's exp/moe/moe_46m_8gpu.sh: same model, global batch (512 x 1024
# tokens per optimizer step, reached with gradient accumulation), precision, optimizer and
# schedule, run by this library's own trainer on synthetic tokens (no dataset is needed).
#
#   bash exp/moe/moe_46m_8gpu.sh [steps] [experts] [capacity_factor] [top_k] [loss_weight] [micro_batch]
set -e
STEPS=${1:-20000}
EXPERTS=${2:-64}
CAPACITY_FACTOR=${3:-16384}
TOP_K=${4:-1}
LOSS_WEIGHT=${5:-0.1}
MICRO_BATCH=${6:-64}
GPUS=${GPUS:-8}
cd "$(dirname "$0")/../.."
python -m torch.distributed.run --nnodes=1 --nproc-per-node "$GPUS" --master-addr 127.0.0.1 --master-port 29500 \
    -m megablocks_b200.train --preset dmoe-46m --steps "$STEPS" --experts "$EXPERTS" --top-k "$TOP_K" \
    --loss-weight "$LOSS_WEIGHT" --micro-batch "$MICRO_BATCH" --global-batch 512 --precision fp16 \
    --optimizer adam --lr 1.5e-4 --min-lr 1e-5 --init-std 0.01 --capacity-factor "$CAPACITY_FACTOR" "${@:7}"
