#!/usr/bin/env bash
# One process per GPU on one node:  scripts/launch_single_node.sh <config-name> [N_GPUS] [overrides...]
set -euo pipefail
CONFIG="${1:?config name}"; shift
NGPU="${1:-8}"; [ $# -gt 0 ] && shift || true
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
set -a; source "$HERE/env/nccl.env"; set +a
export RUN_ID="${RUN_ID:-$(date -u +%Y%m%dT%H%M%SZ)}"
exec python -m torch.distributed.run --standalone --local-addr 127.0.0.1 --nnodes=1 --nproc-per-node="$NGPU" \
  -m open_transformers_b200.cli.train --config-name "$CONFIG" "run.run_id=$RUN_ID" "run.nproc_per_node=$NGPU" "$@"
