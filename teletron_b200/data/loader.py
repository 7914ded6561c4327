"""DataLoader construction (``teletron/core/data_loader.py:10-49``): Megatron-style samplers over a
``torch`` DataLoader with pinned memory; the data-parallel rank/size can be overridden so an encoder
rank can build the loader *of the consumer it serves* (``teletron/training/training.py:271-336``)."""

from __future__ import annotations

from typing import Optional

import torch
from torch.utils.data import DataLoader

from ..parallel import state as ps
from .samplers import PretrainingRandomSampler, PretrainingSampler


def build_pretraining_data_loader(dataset, consumed_samples: int, micro_batch_size: int = 1,
                                  dataloader_type: str = "single", num_workers: int = 1, seed: int = 1234,
                                  dp_rank: Optional[int] = None, dp_size: Optional[int] = None):
    if dataset is None:
        return None
    dp_rank = ps.get_data_parallel_rank() if dp_rank is None else dp_rank
    dp_size = ps.get_data_parallel_world_size() if dp_size is None else dp_size
    if dataloader_type == "single":
        sampler = PretrainingSampler(len(dataset), consumed_samples, micro_batch_size, dp_rank, dp_size)
    elif dataloader_type == "cyclic":
        sampler = PretrainingRandomSampler(len(dataset), consumed_samples, micro_batch_size, dp_rank, dp_size, seed)
    elif dataloader_type == "external":
        return dataset
    else:
        raise ValueError(f"{dataloader_type} dataloader type is not supported")
    return DataLoader(dataset, batch_sampler=sampler, num_workers=num_workers,
                      pin_memory=torch.cuda.is_available(), persistent_workers=num_workers > 0)
