#!/bin/bash
# Usage: ./mpirun_terapipe_new.sh N_NODES N_GPUS_PER_NODE MODEL_PARALLEL_SIZE PIPELINE_PARALLEL_SIZE \
#          MODEL BATCH_SIZE N_BATCH_SLICES N_INPUT_SLICES N_STEPS [EXTRA_ARGS...]
# Same arguments as mpirun_terapipe.sh (scalars only) for the module-style driver terapipe.py.
# EXTRA_ARGS: --mixed-precision, --verify save|load, --verify-path DIR
if [ "$#" -lt 9 ]; then echo "$(sed -n 2,5p "$0")"; exit 1; fi
N_NODES=$1; N_GPUS=$2; MP=$3; PP=$4; MODEL=$5; BATCH=$6; NBS=$7; NIS=$8; N_STEPS=$9
shift 9
if [ "$N_NODES" != "1" ]; then echo "single-machine launcher: N_NODES must be 1"; exit 1; fi
HERE="$(cd "$(dirname "$0")" && pwd)"
PYTHON=${PYTHON:-python}
$PYTHON -m terapipe_b200.utils.launcher --nproc "$N_GPUS" ${TERAPIPE_TIME_LIMIT:+--timeout $TERAPIPE_TIME_LIMIT} \
  "$HERE/terapipe.py" 127.0.0.1 -p "${PORT:-7777}" \
  --model "$MODEL" --batch-size "$BATCH" --n-batch-slices "$NBS" --n-input-slices "$NIS" \
  --model-parallel-size "$MP" --pipeline-parallel-size "$PP" --n-steps "$N_STEPS" --use-mpi "$@"
