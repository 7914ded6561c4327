#!/bin/bash
# HF diffusers HunyuanVideo transformer -> TeleTron (Megatron-layout) checkpoint, sharded for tensor parallelism.
# Usage: bash convert_hf2tel.sh <hf_pipeline_root> <save_dir> [tp]
HF_ROOT=${1:?path to the diffusers HunyuanVideo pipeline root}
SAVE=${2:?output directory}
TP=${3:-1}
python -m teletron_b200.convert_ckpt.hunyuan.convert_hunyuanvideo \
    --load-path "${HF_ROOT}/transformer" \
    --hf-ckpt-path "${HF_ROOT}" \
    --save-path "${SAVE}" \
    --target-params-dtype bf16 \
    --target-tensor-model-parallel-size "${TP}" \
    --target-pipeline-model-parallel-size 1
