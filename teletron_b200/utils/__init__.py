"""Planning helpers: memory model of a training step (:mod:`.memory`), measured machine peaks and rooflines (:mod:`.perf`)."""

from .memory import MemoryEstimate, estimate, max_frames, video_tokens  # noqa: F401
from .perf import measured_peaks, roofline_ms  # noqa: F401
