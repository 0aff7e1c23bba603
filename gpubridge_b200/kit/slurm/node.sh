#!/usr/bin/env bash
# One machine's side of a two-machine run without a scheduler (two cloud instances, two
# workstations): run it on both at about the same time.
#
#   machine A:  NODE_RANK=0 MASTER_ADDR=<A's address> OUT=results/pair gpubridge_b200/kit/slurm/node.sh
#   machine B:  NODE_RANK=1 MASTER_ADDR=<A's address> OUT=results/pair gpubridge_b200/kit/slurm/node.sh
#
# Steps, each journalled like the Slurm jobs' (common.sh): network preflight (interface choice,
# round trip, bandwidth, a real Gloo pair); the thirteen-stage check over both machines with each
# machine an island (GPUBRIDGE_SPLIT_TEST=node) over the Gloo bridge and over the native
# multi-stream TCP bridge on the interface the preflight chose; a short all-reduce sweep.
# GPUS: ranks per machine (default: the GPUs PyTorch sees; with KIT_CPU=1, CPU ranks, default 2).
# Results land in $OUT/node<NODE_RANK>; triage and the validation tables read them as they are.
# Role of the reference's mixed-cloud scripts/gpu/mixed/node.sh.
set -uo pipefail
: "${NODE_RANK:?set NODE_RANK to 0 on the first machine and 1 on the second}"
: "${MASTER_ADDR:?set MASTER_ADDR to an address of the first machine that the second can reach}"
HERE=$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)
BASE=${OUT:-results/pair}
OUT="$BASE/node$NODE_RANK"
# shellcheck source=common.sh
. "$HERE/common.sh"

port=${MASTER_PORT:-29560}
if [ "${KIT_CPU:-0}" = 1 ]; then
    export GPUBRIDGE_VENDOR=${GPUBRIDGE_VENDOR:-nvidia}
    gpus=${GPUS:-2}
else
    gpus=${GPUS:-$("$PYTHON" -c 'import torch; print(torch.cuda.device_count())')}
fi
role=worker
[ "$NODE_RANK" != 0 ] || role=master

step preflight "$PYTHON" -m gpubridge_b200.kit.preflight --role "$role" --master-addr "$MASTER_ADDR" \
    --port "$port" --bandwidth-seconds "${PREFLIGHT_SECONDS:-2}" --out "$OUT/preflight"
chosen="$OUT/preflight/preflight-$role.json"
if [ -f "$chosen" ]; then
    ifname=$("$PYTHON" -c "import json,sys; print(json.load(open(sys.argv[1])).get('chosen_ifname') or '')" "$chosen")
    [ -z "$ifname" ] || export GLOO_SOCKET_IFNAME=$ifname GPUBRIDGE_MULTITCP_IFNAME=$ifname
fi

export GPUBRIDGE_SPLIT_TEST=node
launch() {      # launch NAME BRIDGE MODULE ARGS...
    local name=$1 bridge=$2
    shift 2
    GPUBRIDGE_BRIDGE=$bridge step "$name" "$PYTHON" -m torch.distributed.run --nnodes=2 --node-rank="$NODE_RANK" \
        --nproc-per-node="$gpus" --master-addr "$MASTER_ADDR" --master-port "$((port + 1))" "$@"
}
launch check-gloo gloo -m gpubridge_b200.kit.check --out "$BASE/check-gloo" --in-flight-settle 0.5
launch check-multitcp multitcp -m gpubridge_b200.kit.check --out "$BASE/check-multitcp" --in-flight-settle 0.5
launch sweep multitcp -m gpubridge_b200.bench.bench_all_reduce --smallest 64K --largest "${SWEEP_LARGEST:-256M}" \
    --trials 5 --seconds 2 --inner 4 --targets ours --json "$OUT/sweep.json"
finish
