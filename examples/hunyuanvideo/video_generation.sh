#!/bin/bash
# Usage: bash video_generation.sh <base_model_path> <transformer_ckpt_dir> "<prompt>" [ref_frame.pt]
HERE=$(cd "$(dirname "$0")" && pwd)
python "${HERE}/video_generation.py" --base_model_path "$1" --transformer_model_path "$2" --prompt "$3" \
    --ref_frame "${4:-}" --width 1280 --height 720 --num_frames 49 --num_inference_steps 50 \
    --guidance_scale 4.0 --embedded_guidance_scale 1.0 --output_file output.pt
