#!/bin/bash
# Sanity check: 3 dual + 6 single blocks, deterministic inputs, loss = ||prediction||, 10 iterations.  Two parallel
# layouts must print the same loss curve.  Usage: bash run_unified_sanity_check.sh <TP> <CP> [log file]
export PYTORCH_CUDA_ALLOC_CONF=expandable_segments:True
TP=${1:-1}
CP=${2:-1}
LOG=${3:-}
GPUS=${GPUS_PER_NODE:-$((TP * CP))}
export NUM_LAYERS=3
export NUM_SINGLE_LAYERS=6
export FUSED_KERNELS=1
HERE=$(cd "$(dirname "$0")" && pwd)
unset WORLD_SIZE RANK
CMD="python -m torch.distributed.run --nproc_per_node ${GPUS} --nnodes 1 --master_addr 127.0.0.1 --master_port ${MASTER_PORT:-6001} \
    ${HERE}/pretrain_hunyuanvideo.py --micro-batch-size 1 --train-iters 10 --bf16 --lr 1e-5 --lr-decay-style constant \
    --weight-decay 1e-2 --clip-grad 0.0 --recompute-granularity full --recompute-method block --use-distributed-optimizer \
    --tensor-model-parallel-size ${TP} --context-parallel-size ${CP} --dataset-type FakeDataset --num-workers 1 \
    --num-frames ${NUM_FRAMES:-9} --video-resolution ${WIDTH:-640} ${HEIGHT:-368} --sanity-check --log-interval 1 ${EXTRA_ARGS}"
if [ -n "${LOG}" ]; then ${CMD} > "${LOG}" 2>&1; else ${CMD}; fi
