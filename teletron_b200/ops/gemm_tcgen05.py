"""Python side of the tcgen05 GEMM (``csrc/gemm_tcgen05.cu``).

``gemm(a, b, layout, bias, epi, aux)`` computes ``C[M, N]`` in bf16 with fp32 accumulation:

* layout ``"nt"``: ``a [M, K] @ b [N, K]^T``;  ``"nn"``: ``a [M, K] @ b [K, N]``;  ``"tn"``: ``a [K, M]^T @ b [K, N]``.
* ``epi`` 0: ``+ bias``; 1 / 2: ``gelu_erf / gelu_tanh(acc + bias)`` with the pre-activation written to a
  second output; 3 / 4: ``acc * gelu'(aux)`` (activation backward fused into a data-gradient product).

The kernel's waits are bounded; if one runs out it records a status word that :func:`check_status` turns
into :class:`teletron_b200.ops._lib.CommTimeoutError` (the CUDA context stays usable).
"""

from __future__ import annotations

import os
from typing import Dict, Optional, Tuple

import torch

from . import _lib
from ._lib import c_int, c_long, call, ptr, stream

BF16 = torch.bfloat16
_LAYOUTS = {"nt": (0, 0), "nn": (0, 1), "tn": (1, 1)}
# CTA-pair kernel (thread-block cluster of 2, 256 x 256 tiles) for products with at least one tile per pair of SMs;
# TELETRON_B200_GEMM_2CTA=0 keeps everything on the single-CTA kernel
PAIR_KERNEL = os.environ.get("TELETRON_B200_GEMM_2CTA", "1") != "0"
PAIR_MIN_TILES = 74
COUNTERS = {"pair": 0, "single": 0}


def use_pair_kernel(M: int, N: int) -> bool:
    return PAIR_KERNEL and ((M + 255) // 256) * ((N + 255) // 256) >= PAIR_MIN_TILES
_STATUS: Dict[torch.device, torch.Tensor] = {}


def status_tensor(device: torch.device) -> torch.Tensor:
    t = _STATUS.get(device)
    if t is None:
        t = _STATUS[device] = torch.zeros(4, dtype=torch.int32, device=device)
    return t


def check_status(device: Optional[torch.device] = None) -> None:
    """Synchronise and raise if any GEMM / attention launch on ``device`` abandoned a bounded wait."""
    for dev, t in _STATUS.items():
        if device is not None and dev != device:
            continue
        code = int(t[0].item())
        if code:
            t.zero_()
            raise _lib.CommTimeoutError(f"a tcgen05 kernel on {dev} gave up a bounded wait (status {code})")


def _rowmajor(t: torch.Tensor) -> bool:
    return t.dim() == 2 and t.stride(1) == 1 and t.stride(0) >= t.shape[1] and t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0


def _dims(a: torch.Tensor, b: torch.Tensor, layout: str) -> Tuple[int, int, int]:
    if layout == "nt":
        (M, K), (N, K2) = a.shape, b.shape
    elif layout == "nn":
        (M, K), (K2, N) = a.shape, b.shape
    else:
        (K, M), (K2, N) = a.shape, b.shape
    if K != K2:
        raise ValueError(f"contraction mismatch for {layout}: {tuple(a.shape)} x {tuple(b.shape)}")
    return M, N, K


def supported(a: torch.Tensor, b: torch.Tensor, layout: str) -> bool:
    if not (_lib.available() and a.is_cuda and a.dtype == BF16 and b.dtype == BF16 and _rowmajor(a) and _rowmajor(b)):
        return False
    M, N, K = _dims(a, b, layout)
    if N % 8 or K % 8 or (layout == "tn" and M % 8):
        return False
    return M >= 1 and N >= 8 and K >= 8


def gemm(a: torch.Tensor, b: torch.Tensor, layout: str, bias: Optional[torch.Tensor] = None, epi: int = 0,
         aux: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None):
    """Returns ``C`` (and the pre-activation tensor for ``epi`` 1 / 2)."""
    M, N, K = _dims(a, b, layout)
    a_mn, b_mn = _LAYOUTS[layout]
    c = out if out is not None else torch.empty(M, N, dtype=BF16, device=a.device)
    if epi in (1, 2):
        aux = torch.empty(M, N, dtype=BF16, device=a.device)
    elif epi in (3, 4):
        if aux is None or aux.shape != (M, N) or not aux.is_contiguous():
            raise _lib.NativeError("epilogue 3/4 needs a contiguous [M, N] pre-activation tensor")
    if bias is not None:
        bias = _lib.check(bias.contiguous(), BF16, "bias")
    pair = use_pair_kernel(M, N)
    COUNTERS["pair" if pair else "single"] += 1
    call("tt_gemm2_bf16" if pair else "tt_gemm_bf16", ptr(a), ptr(b), ptr(c), ptr(bias), ptr(aux), c_int(M), c_int(N), c_int(K), c_long(a.stride(0)),
         c_long(b.stride(0)), c_long(c.stride(0)), c_int(a_mn), c_int(b_mn), c_int(epi), ptr(status_tensor(a.device)),
         stream())
    return (c, aux) if epi in (1, 2) else c
