"""teletron_b200: a Blackwell (sm_100a) native long-context video-DiT training framework.

Capabilities mirror Tele-AI/TeleTron (HunyuanVideo-style MMDiT training with mixed
data / tensor / Ulysses-context parallelism, activation recompute, a ZeRO-1 AdamW,
a distributed multimodal-encoder service and Megatron-layout checkpoints), but the
architecture is its own: plain ``torch.nn`` modules over a functional op layer whose
GPU implementations are hand-written sm_100a kernels in ``teletron_b200/csrc``.

Unlike the reference (``teletron/__init__.py:1`` imports a monkey-patching adaptor),
importing this package has no side effects on third-party libraries.
"""

__version__ = "0.1.0"

from . import ops  # noqa: F401
