#!/bin/bash
# Usage: ./terapipe_latency_model.sh MODEL N_GPUS BATCH_SIZE N_STEPS [EXTRA_ARGS...]
# Measures the single-layer latency table with tensor parallelism over N_GPUS.  Three passes,
# one per cost ordering of the scan points, so that a pass ended by an out-of-memory point
# leaves its table behind for the next pass to resume from.
if [ "$#" -lt 4 ]; then echo "$(sed -n 2,5p "$0")"; exit 1; fi
MODEL=$1; N_GPUS=$2; BATCH=$3; N_STEPS=$4
shift 4
HERE="$(cd "$(dirname "$0")" && pwd)"
PYTHON=${PYTHON:-python}
for SORT in 0 1 2; do
  $PYTHON -m terapipe_b200.utils.launcher --nproc "$N_GPUS" \
    "$HERE/terapipe_latency_model.py" 127.0.0.1 -p "${PORT:-7777}" \
    --model "$MODEL" --batch-size "$BATCH" --model-parallel-size "$N_GPUS" --n-steps "$N_STEPS" \
    --sort-function "$SORT" --use-mpi "$@"
done
