"""Scalar fields and their decoders (reference: ``ffcv/fields/basics.py``).  The value lives in
the metadata table, so decoding a batch is one gather into the slot's pinned buffer."""
from dataclasses import replace
from typing import Callable, Tuple

import numpy as np

from ..pipeline.allocation_query import AllocationQuery
from ..pipeline.operation import Operation
from ..pipeline.state import State
from .base import ARG_TYPE, Field


class BasicDecoder(Operation):
    def declare_state_and_memory(self, previous_state: State) -> Tuple[State, AllocationQuery]:
        dt = self.field.metadata_type
        return (replace(previous_state, jit_mode=True, shape=(1,), dtype=dt), AllocationQuery((1,), dt))

    def generate_code(self) -> Callable:
        def decode(batch_indices, destination, metadata, storage_state):
            n = len(batch_indices)
            destination[:n, 0] = metadata[batch_indices]
            return destination[:n]
        return decode


class IntDecoder(BasicDecoder):
    pass


class FloatDecoder(BasicDecoder):
    pass


class _ScalarField(Field):
    dtype = None
    decoder = None

    @property
    def metadata_type(self) -> np.dtype:
        return np.dtype(self.dtype)

    @classmethod
    def from_binary(cls, binary):
        return cls()

    def to_binary(self):
        return np.zeros(1, dtype=ARG_TYPE)[0]

    def encode(self, destination, field, malloc):
        destination[0] = field

    def get_decoder_class(self):
        return self.decoder


class IntField(_ScalarField):
    dtype = '<i8'
    decoder = IntDecoder


class FloatField(_ScalarField):
    dtype = '<f8'
    decoder = FloatDecoder
