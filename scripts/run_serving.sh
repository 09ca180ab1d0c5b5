#!/bin/bash
# Start the serving stack (the role of the reference's run_mindie.sh).
#   scripts/run_serving.sh api    MODEL_DIR [PORT] [MAX_NUM_SEQS] [MAX_MODEL_LEN]   OpenAI-style HTTP service: continuous
#                                                                                  batching engine + FastAPI front end
#   scripts/run_serving.sh worker MODEL_DIR [WORLD_SIZE] [GPU_MEM_GB] [CPU_MEM_GB] [BLOCK_SIZE]
#                                 one ModelRunner worker per GPU for an external engine that drives forward() / swap()
set -eu
MODE="${1:?usage: run_serving.sh api|worker MODEL_DIR ...}"
MODEL_DIR="${2:?usage: run_serving.sh api|worker MODEL_DIR ...}"
case "$MODE" in
  api)
    PORT="${3:-8000}"; SEQS="${4:-32}"; LEN="${5:-}"
    exec python -m mindformers_b200.serving.api_server --model_dir "$MODEL_DIR" --port "$PORT" --max_num_seqs "$SEQS" \
      ${LEN:+--max_model_len "$LEN"}
    ;;
  worker)
    WORLD="${3:-1}"; GPU_GB="${4:-40}"; CPU_GB="${5:-8}"; BLOCK="${6:-128}"
    exec python -m torch.distributed.run --nnodes=1 --nproc-per-node="$WORLD" --master-addr 127.0.0.1 --master-port 8128 \
      -m mindformers_b200.serving_worker --model_dir "$MODEL_DIR" --gpu_mem_gb "$GPU_GB" --cpu_mem_gb "$CPU_GB" --block_size "$BLOCK"
    ;;
  *) echo "unknown mode $MODE" >&2; exit 2 ;;
esac
