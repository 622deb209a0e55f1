"""Field interface (reference: ``ffcv/fields/base.py``)."""
from abc import ABC, abstractmethod
from typing import Type

import numpy as np

ARG_TYPE = np.dtype([('', '<u1', 1024)])


class Field(ABC):
    @property
    @abstractmethod
    def metadata_type(self) -> np.dtype:
        raise NotImplementedError

    @staticmethod
    @abstractmethod
    def from_binary(binary):
        raise NotImplementedError

    @abstractmethod
    def to_binary(self):
        raise NotImplementedError

    @abstractmethod
    def encode(self, destination, field, malloc):
        raise NotImplementedError

    @abstractmethod
    def get_decoder_class(self) -> Type:
        raise NotImplementedError
