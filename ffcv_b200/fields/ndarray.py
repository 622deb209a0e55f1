"""Fixed-shape array fields (reference: ``ffcv/fields/ndarray.py``): same stored bytes and field
arguments, so files are interchangeable with the reference's.  The payload of a sample is the
array's bytes in C order at ``metadata[sample]`` (a file offset).

Decoding a batch is a gather of ``batch`` payloads.  Followed by ``ToTensor`` and ``ToDevice`` of
the GPU an image field of the same loader is decoded on, the gather lands in the image batch's
staged bytes and reaches the device in the same transfer (see ``Graph``); on its own it fills the
slot's pinned host buffer as in the reference.
"""
import json
from dataclasses import replace
from typing import Callable, Tuple, Type

import numpy as np
import torch as ch

from ..pipeline.allocation_query import AllocationQuery
from ..pipeline.operation import Operation
from ..pipeline.state import State
from .base import ARG_TYPE, Field

_MAX_DIMS = 32
_ARGS = np.dtype([('shape', '<u8', _MAX_DIMS), ('type_length', '<u8')])


class NDArrayDecoder(Operation):
    """Default decoder of :class:`NDArrayField`."""

    def declare_state_and_memory(self, previous_state: State) -> Tuple[State, AllocationQuery]:
        f = self.field
        return (replace(previous_state, jit_mode=True, shape=tuple(f.shape), dtype=f.dtype),
                AllocationQuery(tuple(f.shape), f.dtype))

    def generate_code(self) -> Callable:
        read = self.memory_read
        nbytes = int(self.field.element_size)

        def decode(batch_indices, destination, metadata, storage_state):
            n = len(batch_indices)
            flat = destination[:n].reshape(n, -1).view(np.uint8)
            for k, sample in enumerate(batch_indices):
                flat[k] = np.asarray(read(metadata[sample], storage_state))[:nbytes]
            return destination[:n]
        return decode


class NDArrayField(Field):
    """Arrays of one numpy dtype and one shape."""

    def __init__(self, dtype: np.dtype, shape: Tuple[int, ...]):
        self.dtype = np.dtype(dtype)
        self.shape = tuple(int(v) for v in shape)
        if len(self.shape) > _MAX_DIMS:
            raise ValueError(f"at most {_MAX_DIMS} dimensions")
        self.element_size = int(self.dtype.itemsize * np.prod(self.shape, dtype=np.int64))

    @property
    def metadata_type(self) -> np.dtype:
        return np.dtype('<u8')

    @staticmethod
    def from_binary(binary) -> Field:
        raw = np.frombuffer(np.asarray(binary).tobytes(), dtype=np.uint8)
        head = raw[:_ARGS.itemsize].view(_ARGS)[0]
        descr = json.loads(raw[_ARGS.itemsize:_ARGS.itemsize + int(head['type_length'])].tobytes().decode('ascii'))
        descr = [tuple(d) for d in descr]
        if len(descr) != 1:
            raise ValueError("NDArrayField stores arrays of a plain dtype")
        dims = [int(v) for v in head['shape']]
        while dims and dims[-1] == 0:
            dims.pop()
        return NDArrayField(np.dtype(descr)['f0'], tuple(dims))

    def to_binary(self):
        out = np.zeros(1, dtype=ARG_TYPE)[0]
        head = np.zeros(1, dtype=_ARGS)
        head['shape'][0][:len(self.shape)] = self.shape
        text = np.frombuffer(json.dumps(self.dtype.descr).encode('ascii'), dtype=np.uint8)
        head['type_length'][0] = len(text)
        packed = np.concatenate([head.view(np.uint8), text])
        out[0][:len(packed)] = packed
        return out

    def encode(self, destination, field, malloc):
        value = np.ascontiguousarray(field, dtype=self.dtype)
        if value.shape != self.shape:
            raise ValueError(f"expected shape {self.shape}, got {value.shape}")
        destination[0], storage = malloc(self.element_size)
        storage[:] = value.reshape(-1).view(np.uint8)

    def get_decoder_class(self) -> Type[Operation]:
        return NDArrayDecoder


class TorchTensorField(NDArrayField):
    """Same storage for torch tensors of one dtype and shape."""

    def __init__(self, dtype: ch.dtype, shape: Tuple[int, ...]):
        super().__init__(ch.zeros(0, dtype=dtype).numpy().dtype, shape)
        self.torch_dtype = dtype

    def encode(self, destination, field, malloc):
        return super().encode(destination, field.numpy(), malloc)
