#!/usr/bin/env bash
#SBATCH --job-name=gpubridge-one-node
#SBATCH --nodes=1
#SBATCH --exclusive
#SBATCH --time=02:00:00
#SBATCH --output=%x-%j.out
# The whole validation runbook on one NVSwitch box: probe, the thirteen-stage check per island
# split and policy, negative init, P2P, numerical gate, stream mutations, all-reduce sweep
# against NCCL, weak scaling.  Submit with the GPUs you want, e.g.
#   OUT=results/one-node sbatch --gres=gpu:8 gpubridge_b200/kit/slurm/one_node.sbatch
# GPUS overrides the GPU count (default: what Slurm gave the node).
set -uo pipefail
HERE=${KIT_SLURM_DIR:-$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)}
OUT=${OUT:-${SLURM_SUBMIT_DIR:-.}/results/${SLURM_JOB_NAME:-one-node}-${SLURM_JOB_ID:-0}}
# shellcheck source=common.sh
. "$HERE/common.sh"

gpus=${GPUS:-${SLURM_GPUS_ON_NODE:-0}}
mode=()
if [ "${KIT_CPU:-0}" = 1 ]; then
    mode=(--cpu)
    export GPUBRIDGE_VENDOR=${GPUBRIDGE_VENDOR:-nvidia}
    [ "$gpus" -gt 0 ] || gpus=2
fi
# The runbook journals its own steps into $OUT/runbook; here it is one step of the job.
only=()
[ -z "${RUNBOOK_ONLY:-}" ] || read -r -a only <<<"--only $RUNBOOK_ONLY"
STEP_TIMEOUT=${JOB_TIMEOUT:-6600} step runbook "$PYTHON" -m gpubridge_b200.kit.runbook \
    --out "$OUT/runbook" --gpus "$gpus" --step-timeout "$STEP_TIMEOUT" "${mode[@]}" "${only[@]}"
finish
