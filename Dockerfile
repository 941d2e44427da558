# B200 (sm_100a) development image: CUDA 12.8+ toolkit with nvcc, PyTorch, and this repository built in place.
FROM nvcr.io/nvidia/pytorch:25.03-py3

WORKDIR /workspace/megablocks_b200
COPY . .
RUN pip install --no-cache-dir pytest numpy && MAX_JOBS=16 python setup.py build_ext --inplace
ENV PYTHONPATH="/workspace/megablocks_b200:${PYTHONPATH}"
