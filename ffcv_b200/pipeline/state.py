"""Pipeline state threaded through ``declare_state_and_memory`` (reference:
``ffcv/pipeline/state.py:8-20``).  ``jit_mode`` is kept for signature compatibility: in this
implementation it means "numpy arrays on the host", and the same two invariants hold."""
from dataclasses import dataclass
from typing import Tuple

import numpy as np
import torch as ch


@dataclass
class State:
    jit_mode: bool
    device: ch.device
    shape: Tuple[int, ...]
    dtype: np.dtype

    def __post_init__(self):
        if self.jit_mode and self.device != ch.device('cpu'):
            raise AssertionError("Can't be in JIT mode and on the GPU")
        if self.jit_mode and isinstance(self.dtype, ch.dtype):
            raise AssertionError("Can't allocate a torch tensor in JIT mode")
