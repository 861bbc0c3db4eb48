#!/bin/bash
# Shared launcher of the example scripts: one process per GPU through torchrun, on one node or on
# several (every node runs the same script with its own NODE_RANK).
#
#   NNODES=2 NODE_RANK=0 MASTER_ADDR=10.0.0.1 bash examples/grpo/grpo_trainer_qwen25_32b.sh
#
# Environment (all optional):
#   GPUS_PER_NODE  GPUs used on this node (default: all visible GPUs)
#   NNODES         number of nodes (default 1)     NODE_RANK  rank of this node (default 0)
#   MASTER_ADDR    address of node 0 (default 127.0.0.1)      MASTER_PORT  (default 29500)
#   LOG_DIR        where the training log goes (default ./logs)
set -euo pipefail

ROOT=$(cd "$(dirname "${BASH_SOURCE[0]}")/.." && pwd)
export PYTHONPATH="$ROOT:${PYTHONPATH:-}"
GPUS_PER_NODE=${GPUS_PER_NODE:-$(nvidia-smi -L 2>/dev/null | wc -l)}
[ "$GPUS_PER_NODE" -gt 0 ] || GPUS_PER_NODE=1
NNODES=${NNODES:-1}
NODE_RANK=${NODE_RANK:-0}
MASTER_ADDR=${MASTER_ADDR:-127.0.0.1}
MASTER_PORT=${MASTER_PORT:-29500}
LOG_DIR=${LOG_DIR:-$ROOT/logs}
umask 0027
mkdir -p "$LOG_DIR"
ulimit -n 32768 2>/dev/null || true

# Build the kernel library once per checkout (seconds; a no-op when it is up to date).
python -m mindspeed_rl_b200.csrc.build > /dev/null

# launch_trainer <cli script> <default recipe> [recipe] [key=value overrides...]
launch_trainer() {
  local script=$1 default_yaml=$2
  shift 2
  local yaml=${1:-$default_yaml}
  [ $# -gt 0 ] && shift
  echo "recipe: $yaml   nodes: $NNODES x $GPUS_PER_NODE GPUs   node rank: $NODE_RANK"
  python -m torch.distributed.run --nnodes "$NNODES" --node-rank "$NODE_RANK" \
    --nproc-per-node "$GPUS_PER_NODE" --master-addr "$MASTER_ADDR" --master-port "$MASTER_PORT" \
    "$ROOT/cli/$script" --config-name "$yaml" "$@" 2>&1 | tee "$LOG_DIR/${yaml}_node${NODE_RANK}.log"
}
