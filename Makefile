# Developer entry points.  WORLD_SIZE ranks of the multi-process tests run on one node
# and rendezvous at 127.0.0.1.
PYTHON ?= python
PYTEST ?= $(PYTHON) -m pytest
WORLD_SIZE ?= 2
MASTER_PORT ?= 26000
EXTRA_ARGS ?=

.PHONY: build test test-gpu test-dist test-dist-gpu bench

build:
	MAX_JOBS=$${MAX_JOBS:-8} $(PYTHON) setup.py build_ext --inplace

# Everything that needs no GPU (multi-process paths run over gloo).
test:
	$(PYTEST) tests -q -m "not gpu" $(EXTRA_ARGS)

# The CUDA kernels against their fp32 PyTorch oracles (one B200).
test-gpu:
	$(PYTEST) tests -q -m gpu $(EXTRA_ARGS)

# Expert-parallel host logic on CPU ranks.
test-dist:
	$(PYTEST) tests/test_expert_parallel_cpu.py tests/test_trainer_cpu.py tests/test_failure_detection.py -q $(EXTRA_ARGS)

# Fused expert-parallel exchange against the NCCL route on 2-4 GPUs.
test-dist-gpu:
	NCCL_NVLS_ENABLE=0 $(PYTEST) tests/test_expert_parallel_gpu.py -q $(EXTRA_ARGS)

bench:
	$(PYTHON) -m torch.distributed.run --nnodes=1 --nproc-per-node $(WORLD_SIZE) --master-addr 127.0.0.1 \
		--master-port $(MASTER_PORT) bench.py --gpus $(WORLD_SIZE)
