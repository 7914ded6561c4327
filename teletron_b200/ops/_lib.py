"""ctypes binding of ``libteletron_b200.so`` (built by :mod:`teletron_b200.build`).

The library exposes a plain C ABI (``csrc/teletron_b200.h``); tensors cross as raw device pointers
plus the current CUDA stream.  Argument validation that needs tensor metadata (dtype, device,
contiguity, alignment) happens here in :func:`check`; shape arithmetic is re-checked on the C side.
"""

from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

_HERE = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
# TELETRON_B200_LIB points at an alternative build of the library (e.g. one compiled with other flags)
LIB_PATH = os.environ.get("TELETRON_B200_LIB") or os.path.join(_HERE, "lib", "libteletron_b200.so")

_lib: Optional[ctypes.CDLL] = None
_err: str = ""

ERRORS = {1: "invalid argument (shape / alignment / size)", 2: "CUDA runtime error",
          3: "device-side wait timed out", 4: "size beyond a compiled-in maximum"}


class NativeError(RuntimeError):
    pass


class CommTimeoutError(NativeError):
    """A bounded device-side wait (peer flag, barrier) ran out; the CUDA context is still usable."""


def _load() -> Optional[ctypes.CDLL]:
    global _lib, _err
    if _lib is not None:
        return _lib
    if not os.path.isfile(LIB_PATH):
        if os.environ.get("TELETRON_B200_AUTOBUILD", "1") == "1":
            try:
                from .. import build as _build
                _build.build()
            except Exception as e:  # pragma: no cover - depends on toolchain
                _err = f"{LIB_PATH} is missing and the automatic build failed: {e}"
                return None
        else:
            _err = f"{LIB_PATH} is missing"
            return None
    try:
        lib = ctypes.CDLL(LIB_PATH)
    except OSError as e:
        _err = str(e)
        return None
    lib.tt_last_cuda_error.restype = ctypes.c_char_p
    _lib = lib
    return lib


def available() -> bool:
    return _load() is not None


def load_error() -> str:
    return _err


def lib() -> ctypes.CDLL:
    l = _load()
    if l is None:
        raise NativeError("native library unavailable: " + _err)
    return l


def ptr(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


_RAW_STREAM = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_CUR_DEVICE = getattr(torch._C, "_cuda_getDevice", None)


def stream() -> ctypes.c_void_p:
    """The current CUDA stream of the current device as a raw handle.  Every native call asks for it, so it goes
    through the two C entry points directly: ``torch.cuda.current_stream()`` resolves its device argument through
    ``device_count()``, which was measured at ~45 us per call (0.7 s over 15 700 native calls of six training steps)."""
    if _RAW_STREAM is not None and _CUR_DEVICE is not None:
        return ctypes.c_void_p(_RAW_STREAM(_CUR_DEVICE()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def check(t: torch.Tensor, dtype: torch.dtype, name: str, device: Optional[torch.device] = None, align: int = 16) -> torch.Tensor:
    """Validate an operand that will be read through a raw pointer."""
    if not t.is_cuda:
        raise NativeError(f"{name}: expected a CUDA tensor")
    if t.dtype != dtype:
        raise NativeError(f"{name}: expected {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise NativeError(f"{name}: expected a contiguous tensor (shape {tuple(t.shape)}, strides {t.stride()})")
    if t.data_ptr() % align:
        raise NativeError(f"{name}: data pointer is not {align}-byte aligned")
    if device is not None and t.device != device:
        raise NativeError(f"{name}: on {t.device}, expected {device}")
    return t


# kernels launched per native call (for the launch counter the benchmark reports)
KERNELS_PER_CALL = {"tt_ln_mod_bwd": 2, "tt_gate_residual_bwd": 2, "tt_rmsnorm_bwd": 2, "tt_qkv_post_bwd": 2, "tt_attn_bwd": 3, "tt_attn_bwd_fused": 3}
LAUNCHES = 0


# Per-phase device time: when switched on, every native call (and every ``phase`` block, used around NCCL collectives and
# optimizer / gradient-sync sections) is bracketed by two CUDA events on the current stream.  Off, it costs one ``is None`` test.
_PROFILE: Optional[dict] = None


def profile_start() -> None:
    global _PROFILE
    _PROFILE = {}


def profile_stop() -> dict:
    """Synchronise and return ``{name: (milliseconds, count)}`` collected since :func:`profile_start`."""
    global _PROFILE
    prof, _PROFILE = _PROFILE or {}, None
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    return {k: (sum(a.elapsed_time(b) for a, b in v), len(v)) for k, v in prof.items()}


def profiling() -> bool:
    return _PROFILE is not None


class phase:
    """``with phase("tp all-reduce"): ...`` - device time of the enclosed work on the current stream, when profiling."""

    def __init__(self, name: str):
        self.name = name
        self.e0 = None

    def __enter__(self):
        if _PROFILE is not None and torch.cuda.is_available():
            self.e0 = torch.cuda.Event(enable_timing=True)
            self.e0.record()
        return self

    def __exit__(self, *exc):
        if self.e0 is not None and _PROFILE is not None:
            e1 = torch.cuda.Event(enable_timing=True)
            e1.record()
            _PROFILE.setdefault(self.name, []).append((self.e0, e1))
        return False


def call(fn_name: str, *args) -> None:
    """Invoke ``tt_<fn_name>`` and raise on a non-zero status."""
    global LAUNCHES
    fn = getattr(lib(), fn_name)
    if _PROFILE is not None:
        with phase(fn_name):
            rc = fn(*args)
    else:
        rc = fn(*args)
    LAUNCHES += KERNELS_PER_CALL.get(fn_name, 1)
    if rc != 0:
        detail = ERRORS.get(rc, "unknown error")
        if rc == 2:
            detail += ": " + (lib().tt_last_cuda_error() or b"").decode()
        if rc == 3:
            raise CommTimeoutError(f"{fn_name}: {detail}")
        raise NativeError(f"{fn_name} failed ({rc}): {detail}")


c_long = ctypes.c_long
c_int = ctypes.c_int
c_float = ctypes.c_float
