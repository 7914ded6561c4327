#!/bin/bash
# HunyuanVideo training.  Usage: bash run_unified.sh <TP> <CP> <num_frames>   (same positional arguments as the
# reference's examples/hunyuanvideo/run_unified.sh).  Multi-node: WORLD_SIZE = number of nodes, RANK = node rank.
export CUDA_DEVICE_MAX_CONNECTIONS=${CUDA_DEVICE_MAX_CONNECTIONS:-8}
export PYTORCH_CUDA_ALLOC_CONF=expandable_segments:True
TP=${1:-1}
CP=${2:-1}
NUM_FRAMES=${3:-33}
GPUS_PER_NODE=${GPUS_PER_NODE:-$(nvidia-smi -L 2>/dev/null | wc -l)}
NNODES=${WORLD_SIZE:-1}
NODE_RANK=${RANK:-0}
MASTER_ADDR=${MASTER_ADDR:-127.0.0.1}
MASTER_PORT=${MASTER_PORT:-6000}
WORLD=$((GPUS_PER_NODE * NNODES))
GBS=$((WORLD / (TP * CP)))
export NUM_LAYERS=${NUM_LAYERS:-20}
export NUM_SINGLE_LAYERS=${NUM_SINGLE_LAYERS:-40}
export FUSED_KERNELS=${FUSED_KERNELS:-1}
HERE=$(cd "$(dirname "$0")" && pwd)
unset WORLD_SIZE RANK
python -m torch.distributed.run --nproc_per_node "${GPUS_PER_NODE}" --nnodes "${NNODES}" --node_rank "${NODE_RANK}" \
    --master_addr "${MASTER_ADDR}" --master_port "${MASTER_PORT}" \
    "${HERE}/pretrain_hunyuanvideo.py" \
    --num-layers 20 --hidden-size 3072 --num-attention-heads 24 --seq-length 512 --max-position-embeddings 4096 \
    --tokenizer-type NullTokenizer --vocab-size 0 \
    --micro-batch-size 1 --global-batch-size "${GBS}" --train-iters "${TRAIN_ITERS:-10}" \
    --weight-decay 1e-2 --init-method-std 0.006 --clip-grad 0.0 --bf16 --lr 1e-5 --lr-decay-style constant \
    --lr-warmup-fraction 0 \
    --recompute-granularity full --recompute-method block --recompute-num-layers 42 --recompute-save-attention \
    --use-distributed-optimizer --no-rope-fusion --distributed-timeout-minutes 60 \
    --tensor-model-parallel-size "${TP}" --context-parallel-size "${CP}" --fused-comm \
    --dataset-type FakeDataset --split 949,50,1 --dataloader-type single --num-workers 1 --num-frames "${NUM_FRAMES}" \
    --video-resolution 1280 720 \
    --tensorboard-queue-size 10 --log-interval 1 --save-interval 10000 --eval-interval 10000 --eval-iters 0 \
    ${EXTRA_ARGS}
