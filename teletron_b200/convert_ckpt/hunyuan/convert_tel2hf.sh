#!/bin/bash
# TeleTron checkpoint (any tensor-parallel size, read from the directory) -> one HF-named state dict.
# Usage: bash convert_tel2hf.sh <tel_ckpt_dir> <save_dir>
LOAD=${1:?TeleTron checkpoint directory (contains latest_checkpointed_iteration.txt)}
SAVE=${2:?output directory}
python -m teletron_b200.convert_ckpt.hunyuan.convert_hunyuanvideo \
    --load-path "${LOAD}" \
    --save-path "${SAVE}" \
    --target-params-dtype bf16 \
    --convert-checkpoint-from-megatron-to-transformers
