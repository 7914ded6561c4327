#!/bin/bash
# Restart wrapper for long runs: relaunches the given training command from its last checkpoint when it ends with the
# step watchdog's exit code (75: a step exceeded --step-timeout-seconds, e.g. a lost encoder rank or a stalled
# collective) or is killed by a signal; any other exit code is final.
#
# Usage: MAX_RESTARTS=5 bash run_with_restart.sh <command> [args...]
#   e.g. MAX_RESTARTS=3 EXTRA_ARGS="--save ckpt --load ckpt --save-interval 200 --step-timeout-seconds 600" \
#        bash run_with_restart.sh bash run_unified.sh 2 4 33
# The command must pass --save and --load pointing at the same directory, so that a relaunch resumes (iteration, optimizer,
# RNG and the diffusion wrapper's step counter are restored; encoder ranks are told the iteration by the handshake).
MAX_RESTARTS=${MAX_RESTARTS:-3}
RESTART_DELAY=${RESTART_DELAY:-10}
attempt=0
while true; do
    "$@"
    rc=$?
    if [ "$rc" -eq 0 ]; then
        exit 0
    fi
    if [ "$rc" -ne 75 ] && [ "$rc" -lt 128 ]; then
        echo "[restart] command failed with exit code $rc: not restarting" >&2
        exit "$rc"
    fi
    attempt=$((attempt + 1))
    if [ "$attempt" -gt "$MAX_RESTARTS" ]; then
        echo "[restart] giving up after $MAX_RESTARTS restarts (last exit code $rc)" >&2
        exit "$rc"
    fi
    echo "[restart] exit code $rc: restart $attempt of $MAX_RESTARTS in ${RESTART_DELAY}s" >&2
    sleep "$RESTART_DELAY"
done
