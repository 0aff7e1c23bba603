#!/usr/bin/env bash
#SBATCH --job-name=gpubridge-two-nodes
#SBATCH --nodes=2
#SBATCH --ntasks-per-node=1
#SBATCH --exclusive
#SBATCH --time=01:00:00
#SBATCH --output=%x-%j.out
# Two boxes.  Steps: network preflight between the two nodes (interface choice, round trip,
# bandwidth, a real Gloo pair); the thirteen-stage check over both nodes as ONE island (same
# vendor: the island library spans the nodes, no bridge); then with GPUBRIDGE_SPLIT_TEST=node -
# each box an island of its own (its GPUs talk over NVLink inside the fused kernels), the
# leaders joined by a host bridge - with the Gloo bridge and with the native multi-stream TCP
# bridge; an all-reduce sweep over the bridged layout.  The split is a relabelling of one
# vendor's GPUs and every record says so.
#   OUT=results/two-nodes sbatch --gres=gpu:8 gpubridge_b200/kit/slurm/two_nodes.sbatch
set -uo pipefail
HERE=${KIT_SLURM_DIR:-$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)}
OUT=${OUT:-${SLURM_SUBMIT_DIR:-.}/results/${SLURM_JOB_NAME:-two-nodes}-${SLURM_JOB_ID:-0}}
# shellcheck source=common.sh
. "$HERE/common.sh"

gpus=${GPUS:-${SLURM_GPUS_ON_NODE:-0}}
if [ "${KIT_CPU:-0}" = 1 ]; then
    export GPUBRIDGE_VENDOR=${GPUBRIDGE_VENDOR:-nvidia}
    [ "$gpus" -gt 0 ] || gpus=2
fi
master=$(first_node)
port=${MASTER_PORT:-29540}

# Each task of an srun is one node; "auto" makes the task on the first node the master.
step preflight srun --ntasks=2 --ntasks-per-node=1 "$PYTHON" -m gpubridge_b200.kit.preflight \
    --role auto --master-addr "$master" --port "$port" --bandwidth-seconds "${PREFLIGHT_SECONDS:-2}" \
    --out "$OUT/preflight"

# The interface the preflight chose carries the bridge.
chosen="$OUT/preflight/preflight-master.json"
if [ -f "$chosen" ]; then
    ifname=$("$PYTHON" -c "import json,sys; print(json.load(open(sys.argv[1])).get('chosen_ifname') or '')" "$chosen")
    [ -z "$ifname" ] || export GLOO_SOCKET_IFNAME=$ifname GPUBRIDGE_MULTITCP_IFNAME=$ifname
fi

launch() {      # launch NAME BRIDGE MODULE ARGS...: one torchrun per node, both in one rendezvous
    local name=$1 bridge=$2
    shift 2
    GPUBRIDGE_BRIDGE=$bridge step "$name" srun --ntasks=2 --ntasks-per-node=1 \
        "$PYTHON" -m torch.distributed.run --nnodes=2 --nproc-per-node="$gpus" \
        --rdzv-backend=c10d --rdzv-endpoint="$master:$((port + 1))" --rdzv-id="${SLURM_JOB_ID:-0}-$name" "$@"
}
launch check-one-island gloo -m gpubridge_b200.kit.check --out "$OUT/check-one-island" --in-flight-settle 0.5
step summary-one-island "$PYTHON" -m gpubridge_b200.kit.summarize "$OUT/check-one-island"
export GPUBRIDGE_SPLIT_TEST=node
launch check-gloo gloo -m gpubridge_b200.kit.check --out "$OUT/check-gloo" --in-flight-settle 0.5
step summary-gloo "$PYTHON" -m gpubridge_b200.kit.summarize "$OUT/check-gloo"
launch check-multitcp multitcp -m gpubridge_b200.kit.check --out "$OUT/check-multitcp" --in-flight-settle 0.5
step summary-multitcp "$PYTHON" -m gpubridge_b200.kit.summarize "$OUT/check-multitcp"
launch sweep multitcp -m gpubridge_b200.bench.bench_all_reduce --smallest 64K --largest "${SWEEP_LARGEST:-256M}" \
    --trials 5 --seconds 2 --inner 4 --targets ours --json "$OUT/sweep.json"
finish
