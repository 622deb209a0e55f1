"""Image normalisation + type conversion (reference: ``ffcv/transforms/normalize.py``).

As in the reference the arithmetic is a 256 x 3 lookup table computed once in float64,
``((v - mean) / std).astype(type)``, and the per-pixel work is a gather.  The gather is the last
step of the fused GPU kernel; standalone it runs the same kernel on a uint8 CUDA batch.
"""
from dataclasses import replace
from typing import Callable, Optional, Tuple

import numpy as np
import torch as ch

from .. import libffcv as L
from ..pipeline.allocation_query import AllocationQuery
from ..pipeline.operation import Operation
from ..pipeline.state import State


def ch_dtype_from_numpy(dtype):
    return ch.from_numpy(np.zeros((), dtype=dtype)).dtype


class NormalizeImage(Operation):
    """Fast normalization and type conversion of uint8 images to a floating point dtype.

    Parameters
    ----------
    mean: np.ndarray
        The mean vector.
    std: np.ndarray
        The standard deviation vector.
    type: np.dtype
        The desired output type for the result as a numpy type (float16 or float32).
    """

    def __init__(self, mean: np.ndarray, std: np.ndarray, type: np.dtype):
        super().__init__()
        mean = np.asarray(mean, dtype=np.float64)
        std = np.asarray(std, dtype=np.float64)
        table = (np.arange(256)[:, None] - mean[None, :]) / std[None, :]
        self.original_dtype = np.dtype(type)
        if self.original_dtype not in (np.dtype(np.float16), np.dtype(np.float32)):
            raise TypeError("NormalizeImage on the GPU path produces float16 or float32")
        self.lookup_table = table.astype(type)
        self.dtype = self.original_dtype
        self.mode = 'gpu'

    def fuse(self, plan) -> bool:
        return plan.set_table(self.lookup_table)

    def declare_state_and_memory(self, previous_state: State) -> Tuple[State, Optional[AllocationQuery]]:
        if previous_state.device.type != 'cuda':
            raise TypeError("NormalizeImage runs on the GPU: place it after an image decoder "
                            "(ffcv_b200 has no CPU pixel path)")
        t = ch_dtype_from_numpy(self.original_dtype)
        return (replace(previous_state, jit_mode=False, dtype=t),
                AllocationQuery(previous_state.shape, t, previous_state.device))

    def generate_code(self) -> Callable:
        from ..pipeline.graph import shared_context
        raw = self.lookup_table.view(np.int16 if self.original_dtype == np.float16 else np.int32)
        tables = {}
        kind = L.OUT_F16_NHWC if self.original_dtype == np.float16 else L.OUT_F32_NHWC

        def normalize_convert(images, result):
            # accepts (B, H, W, 3), or the channels-last (B, 3, H, W) view the reference requires
            as_nchw = images.dim() == 4 and images.shape[1] == 3 and images.shape[3] != 3
            if as_nchw:
                assert images.is_contiguous(memory_format=ch.channels_last), 'Images need to be in channel last'
                images = images.permute(0, 2, 3, 1)
            images = images.contiguous()
            n, h, w, _ = images.shape
            dev = images.device
            if dev not in tables:
                tables[dev] = ch.from_numpy(raw.copy()).to(dev)
            out = result[:n].view(-1)[:n * h * w * 3].view(n, h, w, 3)
            params = np.zeros((n, 4), dtype=np.int32)
            params[:, 2] = h
            params[:, 3] = w
            plan = L.make_plan(h, w, 0, kind, [], tables[dev].data_ptr())
            shared_context(dev).transform_device(ch.cuda.current_stream(dev).cuda_stream, images.data_ptr(),
                                                 n, h, w, plan, params, out.data_ptr())
            return out.permute(0, 3, 1, 2) if as_nchw else out
        return normalize_convert
