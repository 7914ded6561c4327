"""Sequence padding for Ulysses context parallelism.

The video token count is padded up to a multiple of the context-parallel size before
the sequence split; pad tokens are dropped again right before attention and re-added
after it (reference: ``teletron/core/context_parallel/pad.py:17-52``).  The reference
keeps the two lengths in module globals; here they live in an explicit
:class:`SeqPad` value that the model threads through its blocks, and the global-style
helpers are kept as thin wrappers for API parity.
"""

from __future__ import annotations

import dataclasses
from typing import Optional

import torch
import torch.nn.functional as F


@dataclasses.dataclass(frozen=True)
class SeqPad:
    origin: int   # true number of video tokens
    target: int   # padded to a multiple of the context-parallel size

    @staticmethod
    def for_length(length: int, cp: int) -> "SeqPad":
        target = (length + cp - 1) // cp * cp
        return SeqPad(origin=length, target=target)

    @property
    def pad(self) -> int:
        return self.target - self.origin

    def add(self, x: torch.Tensor, dim: int) -> torch.Tensor:
        n = self.target - x.size(dim)
        if n <= 0:
            return x
        spec = [0] * (2 * x.dim())
        spec[-(2 * dim + 1)] = n
        return F.pad(x, spec)

    def remove(self, x: torch.Tensor, dim: int) -> torch.Tensor:
        if x.size(dim) == self.origin:
            return x
        return x.narrow(dim, 0, self.origin)

    def remove_before_tail(self, x: torch.Tensor, tail: int, dim: int) -> torch.Tensor:
        """Strip the pad that sits between the video tokens and a ``tail`` of text tokens."""
        if self.pad == 0:
            return x
        body = x.narrow(dim, 0, x.size(dim) - tail).narrow(dim, 0, self.origin)
        return torch.cat([body, x.narrow(dim, x.size(dim) - tail, tail)], dim=dim)


_CURRENT: Optional[SeqPad] = None
_ORIGIN: Optional[int] = None


def set_origin_length(length: int) -> None:
    global _ORIGIN
    _ORIGIN = int(length)


def set_target_length(length: int) -> None:
    global _CURRENT
    if _ORIGIN is None:
        raise ValueError("set_origin_length must be called first")
    _CURRENT = SeqPad(origin=_ORIGIN, target=int(length))


def _cur() -> SeqPad:
    if _CURRENT is None:
        raise ValueError("context-parallel lengths are not set")
    return _CURRENT


def pad_for_context_parallel(tensor: torch.Tensor, dim: int) -> torch.Tensor:
    return _cur().add(tensor, dim)


def remove_pad_for_context_parallel(tensor: torch.Tensor, dim: int) -> torch.Tensor:
    return _cur().remove(tensor, dim)


def remove_pad_with_encoder_for_context_parallel(tensor: torch.Tensor, encoder_length: int, dim: int) -> torch.Tensor:
    return _cur().remove_before_tail(tensor, encoder_length, dim)
