# Shared by the job scripts of this folder: source it, then run every command as a step.
#
#   step NAME CMD...    runs CMD under a time limit (STEP_TIMEOUT seconds, default 1200), with its
#                       output in $OUT/NAME.log and one line in $OUT/steps.jsonl - the journal that
#                       `python -m gpubridge_b200.kit.triage` and `kit.runbook` share.  A failed or
#                       overrunning step is recorded and the job goes on: one bad step never costs
#                       the rest of an allocation.
#   finish              prints the table and exits 1 if any step failed.
#
# KIT_TIMEOUT (default 300) is the process-group timeout the kit programs use; it sits below
# STEP_TIMEOUT so that a stuck collective fails with its own message before the step is killed.
# KIT_CPU=1 runs the same jobs on CPU ranks that name their vendor (for clusters' login nodes
# and for the fake cluster of the tests).
# Role of the reference's scripts/gpu/common.sh (`step`, `limited`).

: "${OUT:?set OUT to the results directory}"
: "${STEP_TIMEOUT:=1200}"
: "${KIT_TIMEOUT:=300}"
: "${PYTHON:=python}"
export KIT_TIMEOUT
mkdir -p "$OUT"
KIT_FAILED=0

kit_root() {
    # the checkout this file lives in: three levels up from kit/slurm
    (cd "$(dirname "${BASH_SOURCE[0]}")/../../.." && pwd)
}
PYTHONPATH="$(kit_root)${PYTHONPATH:+:$PYTHONPATH}"
export PYTHONPATH

step() {
    local name=$1
    shift
    local log="$OUT/$name.log" began code ok seconds
    began=$(date +%s)
    printf '[step] %s ... ' "$name"
    timeout --signal=TERM --kill-after=30 "$STEP_TIMEOUT" "$@" >"$log" 2>&1
    code=$?
    seconds=$(($(date +%s) - began))
    if [ "$code" -eq 124 ] || [ "$code" -eq 137 ]; then
        echo "the step ran past its limit" >>"$log"
        ok=false
        code=null
    elif [ "$code" -eq 0 ]; then
        ok=true
    else
        ok=false
    fi
    printf '{"step": "%s", "ok": %s, "exit_code": %s, "seconds": %s, "log": "%s.log"}\n' \
        "$name" "$ok" "$code" "$seconds" "$name" >>"$OUT/steps.jsonl"
    if [ "$ok" = true ]; then
        echo "ok (${seconds} s)"
    else
        echo "FAILED (${seconds} s)"
        KIT_FAILED=1
    fi
    return 0
}

finish() {
    "$PYTHON" -m gpubridge_b200.kit.triage "$OUT" --max-lines 60 || true
    exit "$KIT_FAILED"
}

# First host of the allocation: where rendezvous and the preflight's master live.
first_node() {
    scontrol show hostnames "${SLURM_JOB_NODELIST:?not inside a Slurm job}" | head -n 1
}
