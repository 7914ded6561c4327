#!/bin/bash
# Parallel-layout equivalence on 4 GPUs: TP1-CP2 on GPUs 0,1 and TP2-CP1 on GPUs 2,3 must print the same loss curve
# (the reference's test/test_scripts/run_test_cases.sh leaves the comparison to the reader; here it is checked).
HERE=$(cd "$(dirname "$0")" && pwd)
ROOT=$(cd "${HERE}/../.." && pwd)
LOG_DIR=${LOG_DIR:-"${ROOT}/logs"}
mkdir -p "${LOG_DIR}"
CUDA_VISIBLE_DEVICES=0,1 MASTER_PORT=6101 bash "${ROOT}/examples/hunyuanvideo/run_unified_sanity_check.sh" 1 2 "${LOG_DIR}/tp1cp2.log" &
CUDA_VISIBLE_DEVICES=2,3 MASTER_PORT=6102 bash "${ROOT}/examples/hunyuanvideo/run_unified_sanity_check.sh" 2 1 "${LOG_DIR}/tp2cp1.log" &
wait
python - "$LOG_DIR" <<'PY'
import re, sys
root = sys.argv[1]
def losses(p):
    return [float(m.group(1)) for m in re.finditer(r"\| loss: ([0-9.E+-]+)", open(p).read())]
a, b = losses(f"{root}/tp1cp2.log"), losses(f"{root}/tp2cp1.log")
assert len(a) == len(b) == 10, (len(a), len(b))
worst = max(abs(x - y) / max(abs(x), 1e-6) for x, y in zip(a, b))
print("max relative loss difference:", worst)
assert worst < 2e-2
PY
