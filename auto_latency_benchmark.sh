#!/bin/bash
# Usage: ./auto_latency_benchmark.sh N_GPUS
# Latency tables and link tables for the models planned on one 8-GPU machine.
N_GPUS=${1:-8}
HERE="$(cd "$(dirname "$0")" && pwd)"
for SPEC in "gpt3-1b 1 8" "gpt3-13b 2 8" "gpt3-44b 4 4"; do
  set -- $SPEC
  "$HERE/terapipe_latency_model.sh" "$1" "$2" "$3" 5
  "$HERE/p2p_comm_latency.sh" "$1" --batch-size "$3"
done
