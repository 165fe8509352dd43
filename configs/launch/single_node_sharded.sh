#!/usr/bin/env bash
# One node, one process per GPU, optimizer state sharded over the ranks (ZeRO-1), fused peer-memory collectives.
# Counterpart of launching the reference with an FSDP2 full-shard Accelerate config: with 180 GB per GPU the bf16
# parameters stay replicated, so only gradients (reduce-scatter) and updated parameters (all-gather) move.
#   usage: configs/launch/single_node_sharded.sh <config.yaml> [--section.key value ...]
set -euo pipefail
NPROC="${NPROC:-$(nvidia-smi -L | wc -l)}"
exec python -m torch.distributed.run --nnodes=1 --nproc-per-node "${NPROC}" --master-addr 127.0.0.1 \
    --master-port "${MASTER_PORT:-29500}" -m deberta_b200 train "$@" --train.distributed.parallelism "${PARALLELISM:-zero}"
