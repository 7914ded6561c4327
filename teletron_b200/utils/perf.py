"""Machine peaks and roofline arithmetic shared by the benchmarks and the training log.

The denominators are measured numbers when the file ``MEASURED_PEAKS.json`` sits at the repository root (a STREAM-style
copy bandwidth and cuBLAS bf16 GEMM throughput, burst and sustained); otherwise the stated fallbacks of an earlier
measurement are used.  NVLink: 770 GB/s per direction is the measured peer-copy bandwidth (900 GB/s nominal).
"""

from __future__ import annotations

import json
import os
from typing import Dict

FALLBACK = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
NVLINK_GBS = 770.0


def measured_peaks() -> Dict[str, float]:
    """``{"hbm_gbs", "bf16_tflops", "bf16_tflops_sustained", "nvlink_gbs", "source"}``."""
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    out = dict(FALLBACK, source="fallback")
    try:
        with open(os.path.join(root, "MEASURED_PEAKS.json")) as f:
            d = json.load(f)
        for k in FALLBACK:
            if k in d:
                out[k] = float(d[k])
        out["source"] = "measured"
    except (OSError, ValueError):
        pass
    out["nvlink_gbs"] = NVLINK_GBS
    return out


def roofline_ms(flops: float = 0.0, hbm_bytes: float = 0.0, nvlink_bytes: float = 0.0, sustained: bool = False) -> float:
    """Target time of a kernel: the slowest of its FLOPs at the GEMM peak, its HBM bytes at the copy bandwidth and the
    bytes that must cross NVLink at the peer-copy bandwidth."""
    p = measured_peaks()
    tf = p["bf16_tflops_sustained" if sustained else "bf16_tflops"]
    return 1e3 * max(flops / (tf * 1e12), hbm_bytes / (p["hbm_gbs"] * 1e9), nvlink_bytes / (p["nvlink_gbs"] * 1e9))
