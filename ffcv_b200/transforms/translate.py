"""Random translation (reference: ``ffcv/transforms/translate.py``)."""
from typing import Tuple

import numpy as np

from ..libffcv import OP_TRANSLATE
from ..pipeline.sampling import sample_translations
from .spatial import SpatialOp


class RandomTranslate(SpatialOp):
    """Translate each image randomly in vertical and horizontal directions up to ``padding``
    pixels; uncovered pixels take ``fill``.

    Parameters
    ----------
    padding : int
        Max number of pixels to translate in any direction.
    fill : tuple
        An RGB color ((0, 0, 0) by default) to fill the area outside the shifted image.
    """
    native_type = OP_TRANSLATE

    def __init__(self, padding: int, fill: Tuple[int, int, int] = (0, 0, 0)):
        super().__init__()
        self.padding = padding
        self.fill = np.array(fill)

    def native_arg(self):
        return int(self.padding)

    def native_fill(self):
        return tuple(int(v) for v in self.fill)

    def sample_params(self, seed, n, height, width, out):
        sample_translations(seed, n, int(self.padding), out)
