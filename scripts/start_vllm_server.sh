#!/usr/bin/env bash
# Starts a vLLM OpenAI-compatible server with sleep mode and the weight-transfer endpoints enabled, for
# the optional `inference_backend: vllm` path.  The native engine needs no server.
set -euo pipefail
MODEL=${1:?usage: start_vllm_server.sh <model-dir> [port] [tp]}
PORT=${2:-8000}
TP=${3:-1}
export VLLM_SERVER_DEV_MODE=1
exec python -m vllm.entrypoints.openai.api_server --model "$MODEL" --port "$PORT" --tensor-parallel-size "$TP" \
  --enable-sleep-mode --gpu-memory-utilization 0.5 --dtype bfloat16
