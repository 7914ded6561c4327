"""Parallel runtime: process-group topology, autograd collectives, CP padding, grad buffers."""

from . import state as parallel_state  # noqa: F401
from .mappings import (  # noqa: F401
    split_forward_gather_backward,
    gather_forward_split_backward,
    ulysses_scatter_heads,
    ulysses_gather_heads,
    copy_to_tensor_model_parallel_region,
    reduce_from_tensor_model_parallel_region,
    gather_from_tensor_model_parallel_region,
)
from .pad import SeqPad  # noqa: F401
