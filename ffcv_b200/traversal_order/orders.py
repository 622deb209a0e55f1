"""Sample orders (reference: ``ffcv/traversal_order/``).

``Sequential`` and ``Random`` behave as the reference's, including the use of torch's
``DistributedSampler`` when ``distributed=True`` (a process group must exist).  ``QuasiRandom``
keeps the reference's page-aware shuffle and, unlike the reference (which raises
``NotImplementedError``, quasi_random.py:54-56), also works distributed: every rank shuffles its
strided share of the indices, which keeps the sharding collective-free.  The index list is first
padded with its own head to a multiple of the world size, as ``DistributedSampler`` does, so every
rank sees the same number of samples and therefore the same number of batches.
"""
from abc import ABC, abstractmethod
from typing import Sequence

import numpy as np
import torch.distributed as dist
from numba import njit
from torch.utils.data import DistributedSampler


class TraversalOrder(ABC):
    def __init__(self, loader):
        self.loader = loader
        self.indices = self.loader.indices
        self.seed = self.loader.seed
        self.distributed = loader.distributed
        self.sampler = None

    @abstractmethod
    def sample_order(self, epoch: int) -> Sequence[int]:
        raise NotImplementedError


class Sequential(TraversalOrder):
    def __init__(self, loader):
        super().__init__(loader)
        if self.distributed:
            self.sampler = DistributedSampler(self.indices, shuffle=False, seed=self.seed, drop_last=False)

    def sample_order(self, epoch: int) -> Sequence[int]:
        if not self.distributed:
            return self.indices
        self.sampler.set_epoch(epoch)
        return self.indices[np.array(list(self.sampler))]


class Random(TraversalOrder):
    def __init__(self, loader):
        super().__init__(loader)
        if self.distributed:
            self.sampler = DistributedSampler(self.indices, shuffle=True, seed=self.seed, drop_last=False)

    def sample_order(self, epoch: int) -> Sequence[int]:
        if not self.distributed:
            generator = np.random.default_rng(self.seed + epoch if self.seed is not None else None)
            return generator.permutation(self.indices)
        self.sampler.set_epoch(epoch)
        return self.indices[np.array(list(self.sampler))]


@njit(cache=True)
def _quasi_random_order(seed, page_to_samples, page_sizes, result, buffer_size):
    # Keeps `buffer_size` pages open, draws the next sample from a random open page
    # (ffcv/traversal_order/quasi_random.py:14-39).
    num_pages = len(page_sizes)
    np.random.seed(seed)
    for page_ix in range(num_pages):
        np.random.shuffle(page_to_samples[page_ix, :page_sizes[page_ix]])
    page_order = np.random.permutation(num_pages)
    consumed = np.zeros_like(page_sizes)
    open_pages = [0]
    open_pages.pop()
    next_page = 0
    for s_ix in range(result.shape[0]):
        while next_page < num_pages and len(open_pages) < buffer_size:
            page = page_order[next_page]
            if page_sizes[page] > 0:
                open_pages.append(page)
            next_page += 1
        pick = np.random.randint(0, len(open_pages))
        page = open_pages[pick]
        result[s_ix] = page_to_samples[page, consumed[page]]
        consumed[page] += 1
        if consumed[page] >= page_sizes[page]:
            open_pages.pop(pick)


class QuasiRandom(TraversalOrder):
    def __init__(self, loader):
        super().__init__(loader)
        page_to_samples = loader.memory_manager.page_to_samples
        if not page_to_samples:
            raise ValueError("Dataset won't benefit from QuasiRandom order, use regular Random")
        indices = np.asarray(self.indices)
        if self.distributed:
            if not dist.is_initialized():
                raise RuntimeError("distributed=True needs an initialised torch.distributed process group")
            world = dist.get_world_size()
            pad = (-len(indices)) % world
            if pad and len(indices):
                indices = np.concatenate([indices, np.resize(indices, pad)])
            indices = indices[dist.get_rank()::world]
        self.my_indices = indices
        values, counts = np.unique(indices, return_counts=True)
        multiplicity = dict(zip(values.tolist(), counts.tolist()))  # > 1 only for padded samples
        first_page = min(page_to_samples.keys())
        num_pages = max(page_to_samples.keys()) - first_page + 1
        width = max(len(v) for v in page_to_samples.values()) * (int(counts.max()) if len(counts) else 1)
        self.page_to_samples_array = np.zeros((num_pages, width), dtype=np.int64)
        self.page_sizes = np.zeros(num_pages, dtype=np.int64)
        for page, content in page_to_samples.items():
            row = page - first_page
            for c in sorted(content):
                for _ in range(multiplicity.get(c, 0)):
                    self.page_to_samples_array[row, self.page_sizes[row]] = c
                    self.page_sizes[row] += 1

    def sample_order(self, epoch: int) -> Sequence[int]:
        seed = (self.seed * 912300 + epoch) % (2 ** 32)
        result = np.zeros(len(self.my_indices), dtype=np.int64)
        _quasi_random_order(seed, self.page_to_samples_array.copy(), self.page_sizes, result,
                            2 * self.loader.batch_size)
        return result
