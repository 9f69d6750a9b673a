#!/bin/bash
# Usage: ./auto_mpirun_dp_slices_evaluation.sh N_GPUS
# Evaluates every planned schedule in dp_results.json on this machine.
N_GPUS=${1:-8}
HERE="$(cd "$(dirname "$0")" && pwd)"
PYTHON=${PYTHON:-python}
$PYTHON - "$HERE/dp_results.json" <<'PY' | while read MODEL INDEX; do "$HERE/mpirun_dp_slices_evaluation.sh" 1 "$N_GPUS" "$MODEL" "$INDEX"; done
import collections, json, sys
count = collections.Counter()
for e in json.load(open(sys.argv[1])):
    print(e["model_name"], count[e["model_name"]])
    count[e["model_name"]] += 1
PY
