#!/bin/bash
# Start the development container with every GPU visible and this checkout mounted.
docker run -it --rm --gpus all --ipc=host --ulimit memlock=-1 --cap-add SYS_ADMIN \
       -v "$(pwd)":/workspace/megablocks_b200 megablocks_b200:latest "$@"
