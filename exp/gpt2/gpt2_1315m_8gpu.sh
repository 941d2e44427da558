#!/bin/bash
# Dense (one expert) GPT-2, 1315m backbone, 8 GPUs, bf16
# Counterpart of the reference's exp/gpt2/gpt2_1315m_8gpu.sh: same model, global batch (512 x 1024
# tokens per optimizer step, reached with gradient accumulation), precision, optimizer and
# schedule, run by this library's own trainer on synthetic tokens (no dataset is needed).
#
#   bash exp/gpt2/gpt2_1315m_8gpu.sh [steps] [experts] [top_k] [loss_weight] [micro_batch]
set -e
STEPS=${1:-100000}
EXPERTS=${2:-1}
TOP_K=${3:-1}
LOSS_WEIGHT=${4:-0.1}
MICRO_BATCH=${5:-16}
GPUS=${GPUS:-8}
cd "$(dirname "$0")/../.."
python -m torch.distributed.run --nnodes=1 --nproc-per-node "$GPUS" --master-addr 127.0.0.1 --master-port 29500 \
    -m megablocks_b200.train --preset dmoe-1315m --steps "$STEPS" --experts "$EXPERTS" --top-k "$TOP_K" \
    --loss-weight "$LOSS_WEIGHT" --micro-batch "$MICRO_BATCH" --global-batch 512 --precision bf16 \
    --optimizer adam --lr 4e-4 --min-lr 4e-5 --init-std 0.02 "${@:6}"
