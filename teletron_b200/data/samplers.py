"""Batch samplers with Megatron's semantics (the reference imports them, ``teletron/core/data_loader.py:7, 22-37``).

``PretrainingSampler``: sequential; data-parallel rank ``r`` takes indices
``[consumed + r*mbs, consumed + (r+1)*mbs)`` of every global batch of ``mbs * dp``.
``PretrainingRandomSampler``: epoch-seeded permutation of this rank's bucket, resumable from
``consumed_samples``.
"""

from __future__ import annotations

import torch


class PretrainingSampler:
    def __init__(self, total_samples: int, consumed_samples: int, micro_batch_size: int, data_parallel_rank: int,
                 data_parallel_size: int, drop_last: bool = True):
        if total_samples <= 0:
            raise ValueError("no samples to consume")
        if data_parallel_rank >= data_parallel_size:
            raise ValueError("data_parallel_rank must be smaller than data_parallel_size")
        self.total_samples, self.consumed_samples = total_samples, consumed_samples
        self.micro_batch_size, self.drop_last = micro_batch_size, drop_last
        self.dp_rank, self.dp_size = data_parallel_rank, data_parallel_size
        self.global_mbs = micro_batch_size * data_parallel_size

    def __len__(self):
        return self.total_samples

    def __iter__(self):
        batch = []
        for idx in range(self.consumed_samples, self.total_samples):
            batch.append(idx)
            if len(batch) == self.global_mbs:
                s = self.dp_rank * self.micro_batch_size
                yield batch[s:s + self.micro_batch_size]
                batch = []
        if batch and not self.drop_last:
            s = self.dp_rank * self.micro_batch_size
            yield batch[s:s + self.micro_batch_size]


class PretrainingRandomSampler:
    def __init__(self, total_samples: int, consumed_samples: int, micro_batch_size: int, data_parallel_rank: int,
                 data_parallel_size: int, seed: int = 1234):
        self.total_samples, self.consumed_samples = total_samples, consumed_samples
        self.micro_batch_size, self.seed = micro_batch_size, seed
        self.dp_rank, self.dp_size = data_parallel_rank, data_parallel_size
        self.global_mbs = micro_batch_size * data_parallel_size
        self.last_batch_size = total_samples % self.global_mbs

    def __len__(self):
        return self.total_samples

    def __iter__(self):
        active = self.total_samples - self.last_batch_size
        epoch = self.consumed_samples // active
        current = self.consumed_samples % active
        bucket = (self.total_samples // self.global_mbs) * self.micro_batch_size
        offset = current // self.dp_size
        start = self.dp_rank * bucket
        g = torch.Generator().manual_seed(self.seed + epoch)
        perm = torch.randperm(bucket, generator=g).tolist()
        batch = []
        for i in perm[offset:]:
            batch.append(start + i)
            if len(batch) == self.micro_batch_size:
                self.consumed_samples += self.global_mbs
                yield batch
                batch = []
