#!/bin/bash
# Peak-memory report of one dMoE layer (forward + backward) on one GPU.
python -m megablocks_b200.layers.memory_test "$@"
