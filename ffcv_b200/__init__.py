"""ffcv_b200: FFCV's decode-and-augment image path on B200 GPUs (sm_100a).

Public surface mirrors ``ffcv``: :class:`Loader`, :class:`DatasetWriter`, ``ffcv_b200.fields``,
``ffcv_b200.fields.decoders``, ``ffcv_b200.transforms``, ``ffcv_b200.pipeline``.
"""
from .loader import Loader, OrderOption
from .writer import DatasetWriter

__version__ = '0.1.0'
__all__ = ['Loader', 'OrderOption', 'DatasetWriter']
