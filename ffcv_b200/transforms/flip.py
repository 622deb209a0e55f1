"""Random horizontal flip (reference: ``ffcv/transforms/flip.py``)."""
from ..libffcv import OP_FLIP
from ..pipeline.sampling import sample_flips
from .spatial import SpatialOp


class RandomHorizontalFlip(SpatialOp):
    """Flip the image horizontally with probability flip_prob.

    Parameters
    ----------
    flip_prob : float
        The probability with which to flip each image in the batch horizontally.
    """
    native_type = OP_FLIP

    def __init__(self, flip_prob: float = 0.5):
        super().__init__()
        self.flip_prob = flip_prob

    def sample_params(self, seed, n, height, width, out):
        sample_flips(seed, n, float(self.flip_prob), out)
