"""Base of the transforms that run as their own kernels on a uint8 ``[B, H, W, 3]`` CUDA batch
(colour jitter, mixup, poisoning): the operations of the reference that cannot be folded into the
decoder's launch because they need whole-image or cross-image information."""
from dataclasses import replace
from typing import Optional, Tuple

import numpy as np
import torch as ch

from ..pipeline.allocation_query import AllocationQuery
from ..pipeline.operation import Operation
from ..pipeline.sampling import batch_seed
from ..pipeline.state import State


class DevicePixelOp(Operation):
    needs_buffer = False

    def __init__(self):
        super().__init__()
        self._seed = int(np.random.randint(0, 2 ** 31 - 1))
        self._epoch, self._batch, self._op = 0, 0, 0
        self.last_draw = None  # the random parameters of the last batch, for inspection and tests

    def begin_batch(self, seed, epoch, batch_ix, op_ix):
        """Called by the pipeline graph before every batch: the random draws of the batch are a
        function of the loader's seed and of where the batch and the operation sit."""
        self._seed, self._epoch, self._batch, self._op = seed, epoch, batch_ix, op_ix

    def next_seed(self):
        s = batch_seed(self._seed, self._epoch, self._batch, 1000 + self._op)
        self._batch += 1  # stand-alone use (no graph): successive calls still draw differently
        return s

    def check_input(self, images):
        if not (isinstance(images, ch.Tensor) and images.is_cuda and images.dtype == ch.uint8 and images.dim() == 4
                and images.shape[3] == 3 and images.is_contiguous()):
            raise TypeError(f"{type(self).__name__} works on contiguous uint8 (B, H, W, 3) CUDA batches as the "
                            "image decoders produce them; ffcv_b200 has no CPU pixel path")

    def declare_state_and_memory(self, previous_state: State) -> Tuple[State, Optional[AllocationQuery]]:
        if previous_state.device.type != 'cuda' or len(previous_state.shape) != 3 or previous_state.shape[2] != 3:
            raise TypeError(f"{type(self).__name__} works on uint8 (H, W, 3) CUDA batches produced by the "
                            "image decoders; ffcv_b200 has no CPU pixel path")
        mem = AllocationQuery(previous_state.shape, ch.uint8, previous_state.device) if self.needs_buffer else None
        return replace(previous_state, jit_mode=False), mem
