"""Shared machinery of the uint8 augmentations (flip, translate, cutout).

Fused into the decoder's launch they only contribute a row of random parameters.  Used on their
own (after an operation that cannot be fused) their ``generate_code`` closure runs the same native
kernel on the uint8 ``[B, H, W, 3]`` CUDA tensor they are given.
"""
from dataclasses import replace
from typing import Callable, Optional, Tuple

import numpy as np
import torch as ch

from .. import libffcv as L
from ..pipeline.allocation_query import AllocationQuery
from ..pipeline.operation import Operation
from ..pipeline.sampling import batch_seed
from ..pipeline.state import State


class SpatialOp(Operation):
    native_type = 0

    def __init__(self):
        super().__init__()
        self._calls = 0
        self._seed = int(np.random.randint(0, 2 ** 31 - 1))

    def native_arg(self):
        return 0

    def native_fill(self):
        return (0, 0, 0)

    def sample_params(self, seed, n, height, width, out):
        raise NotImplementedError

    def fuse(self, plan) -> bool:
        return plan.add_spatial(self.native_type, self.native_arg(), self.native_fill(), self)

    def declare_state_and_memory(self, previous_state: State) -> Tuple[State, Optional[AllocationQuery]]:
        if previous_state.device.type != 'cuda' or len(previous_state.shape) != 3 or previous_state.shape[2] != 3:
            raise TypeError(f"{type(self).__name__} works on uint8 (H, W, 3) CUDA batches produced by the "
                            "image decoders; ffcv_b200 has no CPU pixel path")
        return (replace(previous_state, jit_mode=False),
                AllocationQuery(previous_state.shape, ch.uint8, previous_state.device))

    def generate_code(self) -> Callable:
        from ..pipeline.graph import shared_context

        def apply(images, dst):
            n, h, w, _ = images.shape
            images = images.contiguous()
            params = np.zeros((n, 6), dtype=np.int32)
            params[:, 2] = h
            params[:, 3] = w
            col = np.zeros((n, 2), dtype=np.int32)
            self._calls += 1
            self.sample_params(batch_seed(self._seed, 0, self._calls, 0), n, h, w, col)
            params[:, 4:6] = col
            plan = L.make_plan(h, w, 0, L.OUT_U8_NHWC, [(self.native_type, self.native_arg(), self.native_fill())])
            out = dst[:n]
            ctx = shared_context(images.device)
            ctx.transform_device(ch.cuda.current_stream(images.device).cuda_stream, images.data_ptr(), n, h, w,
                                 plan, params, out.data_ptr())
            return out
        return apply
