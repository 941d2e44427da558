#!/bin/bash
# Token exchange benchmark on all GPUs of this node (NCCL all-to-all against the peer-memory push).
NPROC=${1:-8}
python -m torch.distributed.run --nnodes=1 --nproc-per-node "${NPROC}" --master-addr 127.0.0.1 --master-port 6000 \
       -m megablocks_b200.benchmarks.all_to_all_benchmark
