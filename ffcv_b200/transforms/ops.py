"""General operations (reference: ``ffcv/transforms/ops.py``): conversion to tensors, device
placement, image layout and dtype changes."""
from dataclasses import replace
from typing import Callable, Optional, Tuple

import numpy as np
import torch as ch

from ..pipeline.allocation_query import AllocationQuery
from ..pipeline.operation import Operation
from ..pipeline.state import State


class ToTensor(Operation):
    """Convert from Numpy array to PyTorch Tensor (no-op for data that already is one)."""

    def generate_code(self) -> Callable:
        def to_tensor(inp, dst):
            return inp if isinstance(inp, ch.Tensor) else ch.from_numpy(inp)
        return to_tensor

    def declare_state_and_memory(self, previous_state: State) -> Tuple[State, Optional[AllocationQuery]]:
        dt = previous_state.dtype
        if not isinstance(dt, ch.dtype):
            dt = ch.from_numpy(np.empty((), dtype=dt)).dtype
        return replace(previous_state, jit_mode=False, dtype=dt), None

    def fuse(self, plan) -> bool:
        return plan.decoder is not None


class ToDevice(Operation):
    """Move tensor to device.

    Parameters
    ----------
    device: torch.device
        Device to move to.
    non_blocking: bool
        Asynchronous if copying from CPU to GPU.
    """

    def __init__(self, device, non_blocking=True):
        super().__init__()
        self.device = ch.device(device) if not isinstance(device, ch.device) else device
        self.non_blocking = non_blocking

    def generate_code(self) -> Callable:
        def to_device(inp, dst):
            if inp.device == dst.device:
                return inp
            if len(inp.shape) == 4 and inp.is_contiguous(memory_format=ch.channels_last) \
                    and not inp.is_contiguous():
                dst = dst.reshape(inp.shape[0], inp.shape[2], inp.shape[3], inp.shape[1]).permute(0, 3, 1, 2)
            dst = dst[:inp.shape[0]]
            dst.copy_(inp, non_blocking=self.non_blocking)
            return dst
        return to_device

    def declare_state_and_memory(self, previous_state: State) -> Tuple[State, Optional[AllocationQuery]]:
        return (replace(previous_state, jit_mode=False, device=self.device),
                AllocationQuery(previous_state.shape, dtype=previous_state.dtype, device=self.device))

    def fuse(self, plan) -> bool:
        if plan.decoder is None or self.device.type != 'cuda':
            return False
        dev = self.device if self.device.index is not None else ch.device('cuda', ch.cuda.current_device())
        if plan.device is not None and plan.device != dev:
            return False
        plan.device = dev
        return True


class ToTorchImage(Operation):
    """Change tensor to PyTorch format for images (B x C x H x W).

    Parameters
    ----------
    channels_last : bool
        Use torch.channels_last.
    convert_back_int16 : bool
        Convert to float16.
    """

    def __init__(self, channels_last=True, convert_back_int16=True):
        super().__init__()
        self.channels_last = channels_last
        self.convert_int16 = convert_back_int16
        self.enable_int16conv = False

    def generate_code(self) -> Callable:
        do_conv = self.enable_int16conv

        def to_torch_image(inp: ch.Tensor, dst):
            if do_conv:
                inp = inp.view(dtype=ch.float16)
            inp = inp.permute([0, 3, 1, 2])
            if self.channels_last:
                assert inp.is_contiguous(memory_format=ch.channels_last)
                return inp
            dst[:inp.shape[0]] = inp.contiguous()
            return dst[:inp.shape[0]]
        return to_torch_image

    def declare_state_and_memory(self, previous_state: State) -> Tuple[State, Optional[AllocationQuery]]:
        alloc = None
        H, W, C = previous_state.shape
        new_type = previous_state.dtype
        if new_type is ch.int16 and self.convert_int16:
            new_type = ch.float16
            self.enable_int16conv = True
        if not self.channels_last:
            alloc = AllocationQuery((C, H, W), dtype=new_type, device=previous_state.device)
        return replace(previous_state, shape=(C, H, W), dtype=new_type), alloc

    def fuse(self, plan) -> bool:
        return plan.set_torch_image(self.channels_last)


class Convert(Operation):
    """Convert to target data type.

    Parameters
    ----------
    target_dtype: numpy.dtype or torch.dtype
        Target data type.
    """

    def __init__(self, target_dtype):
        super().__init__()
        self.target_dtype = target_dtype

    def generate_code(self) -> Callable:
        def convert(inp, dst):
            return inp.type(self.target_dtype) if isinstance(inp, ch.Tensor) else inp.astype(self.target_dtype)
        return convert

    def declare_state_and_memory(self, previous_state: State) -> Tuple[State, Optional[AllocationQuery]]:
        return replace(previous_state, dtype=self.target_dtype), None

    def fuse(self, plan) -> bool:
        # uint8 -> float is a table gather with the identity table; a NormalizeImage that follows
        # replaces the table (it indexes with the uint8 value, ffcv/transforms/normalize.py:65)
        if plan.decoder is None or plan.sealed:
            return False
        if self.target_dtype in (ch.float16, np.float16):
            return plan.set_identity_table(np.float16)
        if self.target_dtype in (ch.float32, np.float32):
            return plan.set_identity_table(np.float32)
        return False


class View(Operation):
    """View array using np.view or torch.view."""

    def __init__(self, target_dtype):
        super().__init__()
        self.target_dtype = target_dtype

    def generate_code(self) -> Callable:
        def convert(inp, dst):
            return inp.view(self.target_dtype)
        return convert

    def declare_state_and_memory(self, previous_state: State) -> Tuple[State, Optional[AllocationQuery]]:
        return replace(previous_state, dtype=self.target_dtype, jit_mode=False), None
