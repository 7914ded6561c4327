from .pipeline import DEFAULT_PROMPT_TEMPLATE, HunyuanVideoPipeline, PipelineOutput, flow_sigmas, optimized_scale, save_video_tensor  # noqa: F401
