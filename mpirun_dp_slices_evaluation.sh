#!/bin/bash
# Usage: ./mpirun_dp_slices_evaluation.sh N_NODES N_GPUS_PER_NODE MODEL INDEX [EXTRA_ARGS...]
# Runs entry INDEX of MODEL in dp_results.json with its planned (non-uniform) slices.
if [ "$#" -lt 4 ]; then echo "$(sed -n 2,3p "$0")"; exit 1; fi
N_NODES=$1; N_GPUS=$2; MODEL=$3; INDEX=$4
shift 4
if [ "$N_NODES" != "1" ]; then echo "single-machine launcher: N_NODES must be 1"; exit 1; fi
HERE="$(cd "$(dirname "$0")" && pwd)"
PYTHON=${PYTHON:-python}
$PYTHON -m terapipe_b200.utils.launcher --nproc "$N_GPUS" --timeout "${TERAPIPE_TIME_LIMIT:-500}" \
  "$HERE/dp_slices_evaluation.py" 127.0.0.1 -p "${PORT:-7777}" \
  --model-name "$MODEL" --index "$INDEX" --use-mpi "$@"
