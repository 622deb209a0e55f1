"""Mixup for images and labels (reference: ``ffcv/transforms/mixup.py``;
https://arxiv.org/abs/1710.09412).  The image blend runs on the GPU; the label bookkeeping is a
``[B, 3]`` float32 table built on the host exactly as the reference builds it."""
from dataclasses import replace
from typing import Callable, Optional, Tuple

import numpy as np
import torch as ch

from ..pipeline.allocation_query import AllocationQuery
from ..pipeline.operation import Operation
from ..pipeline.sampling import sample_mixup
from ..pipeline.state import State
from .device_op import DevicePixelOp


def _lambdas(alpha, same_lambda, indices, n):
    # both operations seed with the last sample index of the batch (mixup.py:42, :76), which is
    # what keeps the image and the label pipelines of a batch in step
    lam = np.zeros(n, dtype=np.float64)
    sample_mixup(int(indices[-1]) & 0xFFFFFFFF, float(alpha), bool(same_lambda), lam)
    return lam


class ImageMixup(DevicePixelOp):
    """Mixup for images: image i is blended with image i - 1 of the batch.

    Parameters
    ----------
    alpha : float
        Mixup parameter alpha
    same_lambda : bool
        Whether to use the same value of lambda across the whole batch, or an
        individually sampled lambda per image in the batch
    """
    needs_buffer = True

    def __init__(self, alpha: float, same_lambda: bool):
        super().__init__()
        self.alpha = alpha
        self.same_lambda = same_lambda

    def generate_code(self) -> Callable:
        from ..pipeline.graph import shared_context

        def mixer(images, dst, indices):
            self.check_input(images)
            n = images.shape[0]
            lam = _lambdas(self.alpha, self.same_lambda, indices, n)
            self.last_draw = lam
            out = dst[:n]
            shared_context(images.device).mixup(ch.cuda.current_stream(images.device).cuda_stream,
                                                images.data_ptr(), out.data_ptr(), n, images[0].numel(), lam)
            return out
        mixer.with_indices = True
        return mixer


class LabelMixup(Operation):
    """Mixup for labels. Should be initialized in exactly the same way as :class:`ImageMixup`.
    Produces ``[label, label of the previous sample, lambda]`` per sample as float32."""

    def __init__(self, alpha: float, same_lambda: bool):
        super().__init__()
        self.alpha = alpha
        self.same_lambda = same_lambda

    def generate_code(self) -> Callable:
        def mixer(labels, temp_array, indices):
            labels = np.asarray(labels)
            n = labels.shape[0]
            lam = _lambdas(self.alpha, self.same_lambda, indices, n)
            out = temp_array[:n]
            out[:, 0] = labels[:, 0]
            out[:, 1] = np.roll(labels[:, 0], 1)
            out[:, 2] = lam
            return out
        mixer.with_indices = True
        return mixer

    def declare_state_and_memory(self, previous_state: State) -> Tuple[State, Optional[AllocationQuery]]:
        return (replace(previous_state, shape=(3,), dtype=np.dtype('float32')),
                AllocationQuery((3,), dtype=np.dtype('float32')))


class MixupToOneHot(Operation):
    """Turns the ``[B, 3]`` table of :class:`LabelMixup` (already a tensor) into soft one-hot rows."""

    def __init__(self, num_classes: int):
        super().__init__()
        self.num_classes = num_classes

    def generate_code(self) -> Callable:
        def one_hotter(mixedup_labels, dst):
            dst = dst[:mixedup_labels.shape[0]]
            dst.zero_()
            N = mixedup_labels.shape[0]
            rows = ch.arange(N, device=mixedup_labels.device)
            dst[rows, mixedup_labels[:, 0].long()] = mixedup_labels[:, 2]
            mixedup_labels[:, 2] *= -1
            mixedup_labels[:, 2] += 1
            dst[rows, mixedup_labels[:, 1].long()] = mixedup_labels[:, 2]
            return dst
        return one_hotter

    def declare_state_and_memory(self, previous_state: State) -> Tuple[State, Optional[AllocationQuery]]:
        # Should already be converted to tensor
        assert not previous_state.jit_mode
        return (replace(previous_state, shape=(self.num_classes,)),
                AllocationQuery((self.num_classes,), dtype=previous_state.dtype, device=previous_state.device))
