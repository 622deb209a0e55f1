"""Random brightness, contrast and saturation (reference: ``ffcv/transforms/color_jitter.py``),
as CUDA kernels on the decoded uint8 batch, in place like the reference."""
from typing import Callable

import numpy as np
import torch as ch

from ..pipeline.sampling import sample_jitter
from .device_op import DevicePixelOp

BRIGHTNESS, CONTRAST, SATURATION = 0, 1, 2


class _Jitter(DevicePixelOp):
    kind = BRIGHTNESS

    def __init__(self, magnitude: float, p=0.5):
        super().__init__()
        self.p = p
        self.magnitude = magnitude

    def draw(self, n):
        apply = np.zeros(n, dtype=np.uint8)
        ratio = np.zeros(n, dtype=np.float64)
        sample_jitter(self.next_seed(), n, float(self.p), float(max(0, 1 - self.magnitude)),
                      float(1 + self.magnitude), apply, ratio)
        self.last_draw = (apply, ratio)
        return apply, ratio

    def generate_code(self) -> Callable:
        from ..pipeline.graph import shared_context

        def jitter(images, *_):
            self.check_input(images)
            n, h, w, _c = images.shape
            apply, ratio = self.draw(n)
            shared_context(images.device).color_jitter(ch.cuda.current_stream(images.device).cuda_stream,
                                                       images.data_ptr(), n, h, w, self.kind, apply, ratio)
            return images
        return jitter


class RandomBrightness(_Jitter):
    '''
    Randomly adjust image brightness. Operates on the uint8 image batch.

    Parameters
    ----------
    magnitude : float
        randomly choose brightness enhancement factor on [max(0, 1-magnitude), 1+magnitude]
    p : float
        probability to apply brightness
    '''
    kind = BRIGHTNESS


class RandomContrast(_Jitter):
    '''
    Randomly adjust image contrast. Operates on the uint8 image batch.

    Parameters
    ----------
    magnitude : float
        randomly choose contrast enhancement factor on [max(0, 1-magnitude), 1+magnitude]
    p : float
        probability to apply contrast
    '''
    kind = CONTRAST


class RandomSaturation(_Jitter):
    '''
    Randomly adjust image color balance. Operates on the uint8 image batch.

    Parameters
    ----------
    magnitude : float
        randomly choose color balance enhancement factor on [max(0, 1-magnitude), 1+magnitude]
    p : float
        probability to apply saturation
    '''
    kind = SATURATION
