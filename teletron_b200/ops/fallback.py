"""Policy for the library fallbacks of the op layer (cuBLAS for GEMM shapes the tcgen05 kernel does not take, torch
SDPA / the flash-attention library for attention cases it does not take).

A fallback is legitimate in a unit test on an odd shape, but in training it silently replaces the product by the
baseline.  So every fallback site calls :func:`note`: it is logged once per (site, shape), and in strict mode - which
:func:`teletron_b200.training.pretrain.initialize` switches on unless ``--allow-library-fallback`` is given - it raises.
The reference has no such distinction: all of its GEMMs and its attention are library calls
(``teletron/models/dit/dit_attention.py:65-104, 311-313``).
"""

from __future__ import annotations

import os
import sys
from typing import Dict

_STRICT = os.environ.get("TELETRON_B200_STRICT_KERNELS", "0") == "1"
SEEN: Dict[str, int] = {}


class LibraryFallbackError(RuntimeError):
    pass


def set_strict(on: bool) -> None:
    global _STRICT
    _STRICT = bool(on)


def strict() -> bool:
    return _STRICT


def vector_shaped(*dims: int) -> bool:
    """A product with a dimension below 8 (the modulation vectors: batch-1 GEMV, rank-1 weight gradients) has no tile
    for the tensor-core kernel and is not what the policy is about; such cases go to the library without a note."""
    return min(dims) < 8


def note(site: str, detail: str) -> None:
    key = f"{site}: {detail}"
    n = SEEN.get(key, 0)
    SEEN[key] = n + 1
    if _STRICT:
        raise LibraryFallbackError(f"{key} would run on a library kernel instead of the sm_100a one "
                                   f"(pass --allow-library-fallback to permit this)")
    if n == 0:
        print(f"[teletron_b200] library fallback - {key}", file=sys.stderr, flush=True)
