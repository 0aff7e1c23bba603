#!/usr/bin/env bash
# Submit the kit's jobs and note their ids:
#   gpubridge_b200/kit/slurm/submit.sh [--gpus N] [--out DIR] [one_node] [two_nodes] [-- extra sbatch options]
# With no job named, one_node.  Every job writes into DIR/<job>/ (default results/slurm); the ids
# go to DIR/jobs.txt, one "job id" per line.  Afterwards:
#   python -m gpubridge_b200.kit.triage DIR
set -euo pipefail
here=$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)
gpus=8
out=results/slurm
jobs=()
extra=()
while [ $# -gt 0 ]; do
    case $1 in
    --gpus) gpus=$2; shift 2 ;;
    --out) out=$2; shift 2 ;;
    --) shift; extra=("$@"); break ;;
    one_node | two_nodes) jobs+=("$1"); shift ;;
    *) echo "submit.sh: unknown argument $1" >&2; exit 2 ;;
    esac
done
[ ${#jobs[@]} -gt 0 ] || jobs=(one_node)
mkdir -p "$out"
for job in "${jobs[@]}"; do
    mkdir -p "$out/$job"
    id=$(OUT="$(cd "$out/$job" && pwd)" KIT_SLURM_DIR="$here" sbatch --parsable --gres="gpu:$gpus" \
        --output="$out/$job/slurm-%j.out" --export=ALL "${extra[@]}" "$here/$job.sbatch")
    echo "$job $id" | tee -a "$out/jobs.txt"
done
