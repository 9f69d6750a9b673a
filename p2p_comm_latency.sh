#!/bin/bash
# Usage: ./p2p_comm_latency.sh MODEL [EXTRA_ARGS...]
# Measures the stage-to-stage link (two GPUs of this machine) for MODEL's hidden size.
if [ "$#" -lt 1 ]; then echo "$(sed -n 2,3p "$0")"; exit 1; fi
MODEL=$1
shift 1
HERE="$(cd "$(dirname "$0")" && pwd)"
PYTHON=${PYTHON:-python}
$PYTHON -m terapipe_b200.utils.launcher --nproc 2 "$HERE/p2p_comm_latency.py" 127.0.0.1 -p "${PORT:-14399}" \
  --model "$MODEL" --use-mpi "$@"
