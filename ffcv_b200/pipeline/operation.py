"""The operator contract (reference: ``ffcv/pipeline/operation.py:14-41``).

``declare_state_and_memory`` and ``generate_code`` keep the reference's meaning and call
signatures (decoders: ``f(batch_indices, memory, metadata, storage_state)``; transforms:
``f(previous_result, memory[, batch_indices])``).  One method is added: an operation that the GPU
path can absorb describes itself to the fusion pass through :meth:`fuse`.
"""
from abc import ABC, abstractmethod
from typing import Callable, Optional, Tuple

import numpy as np

from .allocation_query import AllocationQuery
from .state import State


class Operation(ABC):
    def __init__(self):
        self.metadata: np.ndarray = None
        self.memory_read: Callable = None

    def accept_field(self, field):
        self.field = field

    def accept_globals(self, metadata, memory_read):
        self.metadata = metadata
        self.memory_read = memory_read

    @abstractmethod
    def generate_code(self) -> Callable:
        raise NotImplementedError

    def declare_shared_memory(self, previous_state: State) -> Optional[AllocationQuery]:
        return None

    def generate_code_for_shared_state(self) -> Optional[Callable]:
        return None

    @abstractmethod
    def declare_state_and_memory(self, previous_state: State) -> Tuple[State, Optional[AllocationQuery]]:
        raise NotImplementedError

    def fuse(self, plan) -> bool:
        """Adds this operation to a :class:`~ffcv_b200.pipeline.fusion.FusedImagePlan`.  Returns
        False when it cannot be part of the single GPU launch (the default)."""
        return False
