#!/bin/bash
# Multi-process launcher around torchrun, with the calling forms of the reference's msrun wrapper
# (scripts/msrun_launcher.sh:56-63):
#   launcher.sh "<cmd>"                                         8 workers on this node
#   launcher.sh "<cmd>" WORKER_NUM
#   launcher.sh "<cmd>" WORKER_NUM MASTER_PORT LOG_DIR JOIN CLUSTER_TIME_OUT
#   launcher.sh "<cmd>" WORKER_NUM LOCAL_WORKER MASTER_ADDR MASTER_PORT NODE_RANK LOG_DIR JOIN CLUSTER_TIME_OUT
# Rank logs go to $LOG_DIR/worker_N.log; LOG_MF_PATH / MF_LOG_SUFFIX are honoured by the Python logger.
set -u
EXECUTE_ORDER="${1:?usage: launcher.sh \"python run_mindformer.py --config X.yaml ...\" [WORKER_NUM ...]}"
WORKER_NUM=8; LOCAL_WORKER=8; MASTER_ADDR="127.0.0.1"; MASTER_PORT=8118; NODE_RANK=0
LOG_DIR="output/msrun_log"; JOIN="False"; CLUSTER_TIME_OUT=7200
case $# in
  1) ;;
  2) WORKER_NUM=$2; LOCAL_WORKER=$2 ;;
  6) WORKER_NUM=$2; LOCAL_WORKER=$2; MASTER_PORT=$3; LOG_DIR=$4; JOIN=$5; CLUSTER_TIME_OUT=$6 ;;
  9) WORKER_NUM=$2; LOCAL_WORKER=$3; MASTER_ADDR=$4; MASTER_PORT=$5; NODE_RANK=$6; LOG_DIR=$7; JOIN=$8; CLUSTER_TIME_OUT=$9 ;;
  *) echo "expected 1, 2, 6 or 9 arguments, got $#" >&2; exit 1 ;;
esac
NNODES=$(( WORKER_NUM / LOCAL_WORKER ))
mkdir -p "$LOG_DIR"
export LOG_MF_PATH="${LOG_MF_PATH:-$(dirname "$LOG_DIR")/log}"
# strip a leading "python" so torchrun can run the script itself
CMD="${EXECUTE_ORDER#python3 }"; CMD="${CMD#python }"
LAUNCH="python -m torch.distributed.run --nnodes=$NNODES --nproc-per-node=$LOCAL_WORKER --node-rank=$NODE_RANK \
  --master-addr=$MASTER_ADDR --master-port=$MASTER_PORT --log-dir=$LOG_DIR --redirects=3 --tee=0 \
  --rdzv-conf=timeout=$CLUSTER_TIME_OUT $CMD"
echo "Running: $LAUNCH"
if [ "$JOIN" = "True" ] || [ "$JOIN" = "true" ]; then
  $LAUNCH; exit $?
else
  nohup $LAUNCH > "$LOG_DIR/launcher.log" 2>&1 &
  echo "started in the background (pid $!); logs under $LOG_DIR"
fi
