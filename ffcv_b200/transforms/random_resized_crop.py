"""Random resized crop applied after decoding (reference:
``ffcv/transforms/random_resized_crop.py``, ``ffcv/transforms/utils/fast_crop.py``): the same box
sampling and INTER_AREA resize as the random-resized-crop decoder, on a batch that was decoded at
its stored size.  Right after a ``SimpleRGBImageDecoder`` it folds into the decoder's GPU launch;
anywhere else it runs the same kernel on the uint8 CUDA batch it is given."""
from dataclasses import replace
from typing import Callable, Optional, Tuple

import numpy as np
import torch as ch

from .. import libffcv as L
from ..pipeline.allocation_query import AllocationQuery
from ..pipeline.operation import Operation
from ..pipeline.sampling import batch_seed, sample_random_crops
from ..pipeline.state import State


class RandomResizedCrop(Operation):
    """Crop a random portion of image with random aspect ratio and resize it to a given size.

    Parameters
    ----------
    scale : Tuple[float, float]
        Lower and upper bounds for the ratio of random area of the crop.
    ratio : Tuple[float, float]
        Lower and upper bounds for random aspect ratio of the crop.
    size : int
        Side length of the output.
    """

    def __init__(self, scale: Tuple[float, float], ratio: Tuple[float, float], size: int):
        super().__init__()
        self.scale = scale
        self.ratio = ratio
        self.size = size
        self._calls = 0
        self._seed = int(np.random.randint(0, 2 ** 31 - 1))

    def sample_crops(self, seed, heights, widths, out):
        sample_random_crops(seed, heights, widths, np.array(self.scale, dtype=np.float64),
                            np.array(self.ratio, dtype=np.float64), out)

    def fuse(self, plan) -> bool:
        return plan.set_post_crop(self, self.size)

    def declare_state_and_memory(self, previous_state: State) -> Tuple[State, Optional[AllocationQuery]]:
        if previous_state.device.type != 'cuda':
            raise TypeError("RandomResizedCrop works on uint8 CUDA batches produced by the image decoders; "
                            "ffcv_b200 has no CPU pixel path")
        return (replace(previous_state, jit_mode=False, shape=(self.size, self.size, 3)),
                AllocationQuery((self.size, self.size, 3), ch.uint8, previous_state.device))

    def generate_code(self) -> Callable:
        from ..pipeline.graph import shared_context

        def random_resized_crop(images, dst):
            n, h, w, _ = images.shape
            images = images.contiguous()
            crops = np.zeros((n, 4), dtype=np.int32)
            self._calls += 1
            self.sample_crops(batch_seed(self._seed, 0, self._calls, 0), np.full(n, h, np.uint16),
                              np.full(n, w, np.uint16), crops)
            plan = L.make_plan(self.size, self.size, 1, L.OUT_U8_NHWC, [])
            out = dst[:n]
            shared_context(images.device).transform_device(ch.cuda.current_stream(images.device).cuda_stream,
                                                           images.data_ptr(), n, h, w, plan, crops, out.data_ptr())
            return out
        return random_resized_crop
