from .config import HunyuanParams, hunyuan_13b, sanity_config, tiny_config  # noqa: F401
from .model import HunyuanVideoTransformer3DModel  # noqa: F401
from .pipeline import FlowConfig, FlowMatchScheduler, HunyuanPipeline  # noqa: F401
