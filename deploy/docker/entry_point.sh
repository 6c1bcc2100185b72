#!/bin/sh
# MODEL (directory under /models or absolute path) and optional TP_SIZE (GPUs of this node) select what is served.
set -e
MODEL="${MODEL:?set MODEL to a model directory}"
PORT="${PORT:-8080}"
TP_SIZE="${TP_SIZE:-1}"
EXTRA="${SERVER_ARGS:-}"
if [ "$TP_SIZE" -gt 1 ]; then
  exec python -m torch.distributed.run --nnodes=1 --nproc-per-node "$TP_SIZE" --master-addr 127.0.0.1 --master-port 29500 \
       -m deliverance_b200.server --model "$MODEL" --host 0.0.0.0 --port "$PORT" $EXTRA
fi
exec python -m deliverance_b200.server --model "$MODEL" --host 0.0.0.0 --port "$PORT" $EXTRA
