#!/bin/bash
# Dropless MoE, 125m backbone, 8 GPUs, bf16, adam
# Counterpart of the reference's exp/dmoe/dmoe_125m_8gpu.sh: same model, global batch (512 x 1024
# tokens per optimizer step, reached with gradient accumulation), precision, optimizer and
# schedule, run by this library's own trainer on synthetic tokens (no dataset is needed).
#
#   bash exp/dmoe/dmoe_125m_8gpu.sh [steps] [experts] [top_k] [loss_weight] [micro_batch]
set -e
STEPS=${1:-20000}
EXPERTS=${2:-64}
TOP_K=${3:-1}
LOSS_WEIGHT=${4:-0.1}
MICRO_BATCH=${5:-32}
GPUS=${GPUS:-8}
cd "$(dirname "$0")/../.."
python -m torch.distributed.run --nnodes=1 --nproc-per-node "$GPUS" --master-addr 127.0.0.1 --master-port 29500 \
    -m megablocks_b200.train --preset dmoe-125m --steps "$STEPS" --experts "$EXPERTS" --top-k "$TOP_K" \
    --loss-weight "$LOSS_WEIGHT" --micro-batch "$MICRO_BATCH" --global-batch 512 --precision bf16 \
    --optimizer adam --lr 6e-4 --min-lr 6e-5 --init-std 0.01 "${@:6}"
