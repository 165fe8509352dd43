#!/usr/bin/env bash
# One node, one process per GPU, everything replicated, gradients all-reduced (the default multi-GPU mode of the
# reference: DDP). Uses the one-kernel all-reduce over peer memory; --train.distributed.fused_collectives false
# switches to NCCL.
#   usage: configs/launch/single_node_replicated.sh <config.yaml> [--section.key value ...]
set -euo pipefail
NPROC="${NPROC:-$(nvidia-smi -L | wc -l)}"
exec python -m torch.distributed.run --nnodes=1 --nproc-per-node "${NPROC}" --master-addr 127.0.0.1 \
    --master-port "${MASTER_PORT:-29500}" -m deberta_b200 train "$@" --train.distributed.parallelism ddp
