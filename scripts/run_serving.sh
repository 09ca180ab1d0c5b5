#!/bin/bash
# Start one ModelRunner worker per GPU for an external serving engine (the role of the reference's run_mindie.sh):
#   scripts/run_serving.sh MODEL_DIR [WORLD_SIZE] [GPU_MEM_GB] [CPU_MEM_GB] [BLOCK_SIZE]
# Each worker imports mindformers_b200.model_runner.ModelRunner; the engine drives forward()/swap() over its own RPC.
set -eu
MODEL_DIR="${1:?usage: run_serving.sh MODEL_DIR [WORLD_SIZE] [GPU_MEM_GB] [CPU_MEM_GB] [BLOCK_SIZE]}"
WORLD="${2:-1}"; GPU_GB="${3:-40}"; CPU_GB="${4:-8}"; BLOCK="${5:-128}"
exec python -m torch.distributed.run --nnodes=1 --nproc-per-node="$WORLD" --master-addr 127.0.0.1 --master-port 8128 \
  -m mindformers_b200.serving_worker --model_dir "$MODEL_DIR" --gpu_mem_gb "$GPU_GB" --cpu_mem_gb "$CPU_GB" --block_size "$BLOCK"
