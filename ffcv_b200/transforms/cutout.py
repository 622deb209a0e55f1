"""Cutout augmentation, https://arxiv.org/abs/1708.04552 (reference: ``ffcv/transforms/cutout.py``)."""
from typing import Tuple

import numpy as np

from ..libffcv import OP_CUTOUT
from ..pipeline.sampling import sample_cutouts
from .spatial import SpatialOp


class Cutout(SpatialOp):
    """Fill a random ``crop_size`` square of every image with ``fill``.

    Parameters
    ----------
    crop_size : int
        Size of the random square to cut out.
    fill : Tuple[int, int, int], optional
        An RGB color ((0, 0, 0) by default) to fill the cutout square with.
    """
    native_type = OP_CUTOUT

    def __init__(self, crop_size: int, fill: Tuple[int, int, int] = (0, 0, 0)):
        super().__init__()
        self.crop_size = crop_size
        self.fill = np.array(fill)

    def native_arg(self):
        return int(self.crop_size)

    def native_fill(self):
        return tuple(int(v) for v in self.fill)

    def sample_params(self, seed, n, height, width, out):
        sample_cutouts(seed, n, int(height), int(width), int(self.crop_size), out)
