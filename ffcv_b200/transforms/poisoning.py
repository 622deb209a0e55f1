"""Poison images by adding a mask (reference: ``ffcv/transforms/poisoning.py``), on the GPU."""
from typing import Callable

import numpy as np
import torch as ch

from .device_op import DevicePixelOp


class Poison(DevicePixelOp):
    """Poison specified images by adding a mask with given opacity.

    Parameters
    ----------
    mask : ndarray
        The mask to apply to each image, (H, W, 3).
    alpha: ndarray
        The opacity of the mask, (H, W).
    indices : Sequence[int]
        The indices of images that should have the mask applied.
    clamp : Tuple[int, int]
        Clamps the final pixel values between these two values (default: (0, 255)).
    """

    def __init__(self, mask: np.ndarray, alpha: np.ndarray, indices, clamp=(0, 255)):
        super().__init__()
        self.mask = mask
        self.indices = np.sort(indices)
        self.clamp = clamp
        self.alpha = alpha
        self._dev = {}

    def generate_code(self) -> Callable:
        from ..pipeline.graph import shared_context
        # poisoning.py:38-39: the opacity repeated over the channels, the mask pre-multiplied by it
        alpha = np.repeat(np.asarray(self.alpha)[:, :, None], 3, axis=2)
        mask = np.ascontiguousarray(np.asarray(self.mask).astype('float') * alpha, dtype=np.float64)
        one_minus = np.ascontiguousarray(1 - alpha, dtype=np.float64)
        to_poison = self.indices

        def poison(images, temp_array, indices):
            self.check_input(images)
            n = images.shape[0]
            if tuple(images.shape[1:]) != mask.shape:
                raise ValueError(f"Poison mask of shape {mask.shape} applied to images of shape {tuple(images.shape[1:])}")
            key = images.device.index
            if key not in self._dev:
                self._dev[key] = (ch.from_numpy(one_minus).to(images.device), ch.from_numpy(mask).to(images.device))
            oma_dev, mask_dev = self._dev[key]
            indices = np.asarray(indices)
            position = np.searchsorted(to_poison, indices)
            apply = np.zeros(n, dtype=np.uint8)
            inside = position < len(to_poison)
            apply[inside] = to_poison[position[inside]] == indices[inside]
            self.last_draw = apply
            if apply.any():
                shared_context(images.device).poison(ch.cuda.current_stream(images.device).cuda_stream,
                                                     images.data_ptr(), n, images[0].numel(), apply,
                                                     oma_dev.data_ptr(), mask_dev.data_ptr(), self.clamp[0], self.clamp[1])
            return images
        poison.with_indices = True
        return poison
