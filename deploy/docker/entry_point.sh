#!/bin/sh
# MODEL (directory under /models or absolute path) and optional TP_SIZE (GPUs of this node) select what is served.
set -e
CONFIG="${CONFIG:-}"   # optional .properties / .json configuration (models, KV cache, auth; see example-config.json); replaces MODEL
if [ -n "$CONFIG" ]; then
  exec python -m deliverance_b200.server --config "$CONFIG" --models-root "${MODELS_ROOT:-/models}" --host 0.0.0.0 ${SERVER_ARGS:-}
fi
MODEL="${MODEL:?set MODEL to a model directory (or CONFIG to a .properties file)}"
PORT="${PORT:-8080}"
TP_SIZE="${TP_SIZE:-1}"
EXTRA="${SERVER_ARGS:-}"
if [ "$TP_SIZE" -gt 1 ]; then
  # the rank supervisor starts one process per GPU and restarts the whole group when a rank dies or stops reporting
  # (SUPERVISE=0 falls back to a plain torchrun launch)
  if [ "${SUPERVISE:-1}" = "1" ]; then
    exec python -m deliverance_b200.parallel.cluster --nproc "$TP_SIZE" --no-exit-ok --max-restarts "${MAX_RESTARTS:-5}" \
         --hang-timeout "${HANG_TIMEOUT:-120}" --start-timeout "${START_TIMEOUT:-1800}" --status-file /tmp/deliverance-cluster.json -- \
         python -m deliverance_b200.server --model "$MODEL" --host 0.0.0.0 --port "$PORT" $EXTRA
  fi
  exec python -m torch.distributed.run --nnodes=1 --nproc-per-node "$TP_SIZE" --master-addr 127.0.0.1 --master-port 29500 \
       -m deliverance_b200.server --model "$MODEL" --host 0.0.0.0 --port "$PORT" $EXTRA
fi
exec python -m deliverance_b200.server --model "$MODEL" --host 0.0.0.0 --port "$PORT" $EXTRA
