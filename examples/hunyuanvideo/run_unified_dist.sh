#!/bin/bash
# Training with the distributed multimodal-encoder service: the last ENC ranks run the VAE + text encoders and
# stream encoded samples to the DiT ranks.  Usage: bash run_unified_dist.sh <TP> <CP> <num_frames> [ENC]
# (the reference's script uses $3 for both the process count and the frame count; here they are separate).
export PYTORCH_CUDA_ALLOC_CONF=expandable_segments:True
TP=${1:-2}
CP=${2:-3}
NUM_FRAMES=${3:-33}
ENC=${4:-2}
GPUS_PER_NODE=${GPUS_PER_NODE:-$(nvidia-smi -L 2>/dev/null | wc -l)}
MASTER_ADDR=${MASTER_ADDR:-127.0.0.1}
MASTER_PORT=${MASTER_PORT:-6000}
DIT=$((GPUS_PER_NODE - ENC))
GBS=$((DIT / (TP * CP)))
export NUM_LAYERS=${NUM_LAYERS:-20}
export NUM_SINGLE_LAYERS=${NUM_SINGLE_LAYERS:-40}
HERE=$(cd "$(dirname "$0")" && pwd)
unset WORLD_SIZE RANK
python -m torch.distributed.run --nproc_per_node "${GPUS_PER_NODE}" --nnodes 1 --master_addr "${MASTER_ADDR}" \
    --master_port "${MASTER_PORT}" "${HERE}/pretrain_hunyuanvideo.py" \
    --micro-batch-size 1 --global-batch-size "${GBS}" --train-iters "${TRAIN_ITERS:-10}" \
    --weight-decay 1e-2 --init-method-std 0.006 --clip-grad 0.0 --bf16 --lr 1e-5 --lr-decay-style constant \
    --recompute-granularity full --recompute-method block --recompute-save-attention --use-distributed-optimizer \
    --distributed-timeout-minutes 60 --tensor-model-parallel-size "${TP}" --context-parallel-size "${CP}" --fused-comm \
    --distributed-vae --distributed-vae-world-size "${ENC}" \
    --dataset-type FakeDataset --dataloader-type single --num-workers 1 --num-frames "${NUM_FRAMES}" \
    --video-resolution 1280 720 --log-interval 1 ${EXTRA_ARGS}
