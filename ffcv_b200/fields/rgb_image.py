"""RGB image field and its decoders (reference: ``ffcv/fields/rgb_image.py``).

Same classes, constructor arguments and metadata layout as the reference.  What differs is where
the pixels are produced: a decoder here never touches pixels on the CPU.  It ships the stored
bytes (JPEG stream, or the rows of a raw image its crop touches) to the GPU, where
``libffcv_b200.so`` decodes, crops and resizes them; its result is a uint8 ``[B, H, W, 3]`` CUDA
tensor instead of a host array.
"""
from abc import ABCMeta, abstractmethod
from dataclasses import replace
from typing import Callable, Tuple, Type

import cv2
import numpy as np
import torch as ch

from ..pipeline.allocation_query import AllocationQuery
from ..pipeline.operation import Operation
from ..pipeline.sampling import sample_center_crops, sample_random_crops
from ..pipeline.state import State
from .base import ARG_TYPE, Field

IMAGE_MODES = {'jpg': 0, 'raw': 1}


def encode_jpeg(numpy_image, quality, restart_interval=0):
    """``cv2.imencode('.jpg', BGR, [IMWRITE_JPEG_QUALITY, q])`` as rgb_image.py:26-34 does:
    baseline, 4:2:0, standard Huffman tables, no restart markers -- unless ``restart_interval``
    (in MCUs) asks for them."""
    bgr = cv2.cvtColor(numpy_image, cv2.COLOR_RGB2BGR)
    flags = [int(cv2.IMWRITE_JPEG_QUALITY), quality]
    if restart_interval:
        flags += [int(cv2.IMWRITE_JPEG_RST_INTERVAL), int(restart_interval)]
    ok, result = cv2.imencode('.jpg', bgr, flags)
    if not ok:
        raise ValueError("Impossible to encode image in jpeg")
    return result.reshape(-1)


def resizer(image, target_resolution):
    """Write-time downscale so that the longer side is ``target_resolution`` (rgb_image.py:37-45)."""
    if target_resolution is None:
        return image
    original_size = np.array([image.shape[1], image.shape[0]])
    ratio = target_resolution / original_size.max()
    if ratio < 1:
        new_size = (ratio * original_size).astype(int)
        image = cv2.resize(image, tuple(new_size), interpolation=cv2.INTER_AREA)
    return image


def _cuda_device():
    if not ch.cuda.is_available():
        raise RuntimeError("ffcv_b200 decodes on the GPU and has no CPU fallback: no CUDA device is visible")
    return ch.device('cuda', ch.cuda.current_device())


class SimpleRGBImageDecoder(Operation):
    """Decoder for datasets whose images all have the same resolution; passes them through as
    stored (reference: rgb_image.py:84-139)."""

    def __init__(self):
        super().__init__()

    def _extent(self):
        widths, heights = self.metadata['width'], self.metadata['height']
        return int(heights.min()), int(heights.max()), int(widths.min()), int(widths.max())

    def output_shape(self):
        hmin, hmax, wmin, wmax = self._extent()
        if hmin != hmax or wmin != wmax:
            raise TypeError("SimpleRGBImageDecoder only supports constant image,\n"
                            "consider RandomResizedCropRGBImageDecoder or CenterCropRGBImageDecoder\n"
                            "instead.")
        return hmax, wmax

    def declare_state_and_memory(self, previous_state: State) -> Tuple[State, AllocationQuery]:
        h, w = self.output_shape()
        device = _cuda_device()
        return (replace(previous_state, jit_mode=False, device=device, shape=(h, w, 3), dtype=ch.uint8),
                AllocationQuery((h, w, 3), ch.uint8, device))

    def sample_crops(self, seed, heights, widths, out):
        out[:, 0] = 0
        out[:, 1] = 0
        out[:, 2] = heights
        out[:, 3] = widths

    def fuse(self, plan) -> bool:
        h, w = self.output_shape()
        return plan.set_decoder(self, h, w, resize=False)

    def generate_code(self) -> Callable:
        from ..pipeline.graph import standalone_decoder
        return standalone_decoder(self)


class ResizedCropRGBImageDecoder(SimpleRGBImageDecoder, metaclass=ABCMeta):
    """Crop then INTER_AREA-resize to ``output_size`` (reference: rgb_image.py:142-217).

    ``dct_downscale`` (not in the reference, off by default): decode a JPEG sample at 1/2, 1/4 or 1/8
    scale -- the ``scale_num / scale_denom`` of the reference's ``imdecode``
    (libffcv/libffcv.cpp:59,89-90), which its decoders always leave at 1/1 -- whenever the sample's
    crop box still has at least ``output_size`` pixels at that scale, and resize from the scaled
    image.  The scaled decode equals libjpeg-turbo's bit for bit, but a crop resized from it is not
    the crop resized from the full decode, so the pixels are no longer the reference's."""

    def __init__(self, output_size, dct_downscale=False):
        super().__init__()
        self.output_size = output_size
        self.dct_downscale = bool(dct_downscale)

    def output_shape(self):
        return int(self.output_size[0]), int(self.output_size[1])

    def fuse(self, plan) -> bool:
        h, w = self.output_shape()
        if not plan.set_decoder(self, h, w, resize=True):
            return False
        plan.dct_scale = -1 if self.dct_downscale else 0
        return True

    @property
    @abstractmethod
    def get_crop_generator(self):
        raise NotImplementedError


class RandomResizedCropRGBImageDecoder(ResizedCropRGBImageDecoder):
    """Random-resized-crop decoder (reference: rgb_image.py:220-242).

    Parameters
    ----------
    output_size : Tuple[int]
        The desired resized resolution of the images
    scale : Tuple[float]
        The range of possible ratios (in area) than can randomly sampled
    ratio : Tuple[float]
        The range of potential aspect ratios that can be randomly sampled
    """

    def __init__(self, output_size, scale=(0.08, 1.0), ratio=(0.75, 4 / 3), dct_downscale=False):
        super().__init__(output_size, dct_downscale)
        self.scale = scale
        self.ratio = ratio

    def sample_crops(self, seed, heights, widths, out):
        sample_random_crops(seed, heights, widths, np.array(self.scale, dtype=np.float64),
                            np.array(self.ratio, dtype=np.float64), out)

    @property
    def get_crop_generator(self):
        from ..pipeline.sampling import _random_crop
        return _random_crop


class CenterCropRGBImageDecoder(ResizedCropRGBImageDecoder):
    """Centre-crop decoder (reference: rgb_image.py:245-265).

    Parameters
    ----------
    output_size : Tuple[int]
        The desired resized resolution of the images
    ratio: float
        ratio of (crop size) / (min side length)
    """

    def __init__(self, output_size, ratio, dct_downscale=False):
        super().__init__(output_size, dct_downscale)
        self.scale = None
        self.ratio = ratio

    def sample_crops(self, seed, heights, widths, out):
        sample_center_crops(heights, widths, float(self.ratio), out)

    @property
    def get_crop_generator(self):
        def get_center_crop(height, width, _, ratio):
            c = int(ratio * min(height, width))
            return (height - c) // 2, (width - c) // 2, c, c
        return get_center_crop


class RGBImageField(Field):
    """RGB image field; arguments and stored bytes as the reference's (rgb_image.py:268-365).

    ``write_mode`` is 'raw', 'jpg', 'smart' or 'proportion'; ``max_resolution`` bounds the longer
    side at write time; ``jpeg_quality`` and ``compress_probability`` as in the reference.

    ``jpeg_restart_interval`` (not in the reference; a write-time choice that is not stored in the
    field's arguments) makes the encoder emit a restart marker every that many MCUs.  The file
    stays an ordinary ``.beton`` that the reference reads as well (restart markers are part of
    baseline JPEG); here such streams need no speculative decoding: every interval is decoded by
    its own GPU thread.  4 to 8 MCUs cost about 1 % of file size.
    """

    def __init__(self, write_mode='raw', max_resolution: int = None, smart_threshold: int = None,
                 jpeg_quality: int = 90, compress_probability: float = 0.5,
                 jpeg_restart_interval: int = 0) -> None:
        self.write_mode = write_mode
        self.smart_threshold = smart_threshold
        self.max_resolution = max_resolution
        self.jpeg_quality = int(jpeg_quality)
        self.proportion = compress_probability
        self.jpeg_restart_interval = int(jpeg_restart_interval)

    @property
    def metadata_type(self) -> np.dtype:
        return np.dtype([('mode', '<u1'), ('width', '<u2'), ('height', '<u2'), ('data_ptr', '<u8')])

    def get_decoder_class(self) -> Type[Operation]:
        return SimpleRGBImageDecoder

    @staticmethod
    def from_binary(binary) -> Field:
        return RGBImageField()

    def to_binary(self):
        return np.zeros(1, dtype=ARG_TYPE)[0]

    def encode_jpeg(self, image):
        return encode_jpeg(image, self.jpeg_quality, self.jpeg_restart_interval)

    def choose_mode(self, image):
        """Returns ('jpg' | 'raw', jpeg bytes or None)."""
        mode, as_jpg = self.write_mode, None
        if mode == 'smart':
            as_jpg = self.encode_jpeg(image)
            mode = 'raw'
            if self.smart_threshold is not None and image.nbytes > self.smart_threshold:
                mode = 'jpg'
        elif mode == 'proportion':
            mode = 'jpg' if np.random.rand() < self.proportion else 'raw'
        return mode, as_jpg

    def encode(self, destination, image, malloc):
        if hasattr(image, 'convert') and not isinstance(image, np.ndarray):
            image = np.array(image)  # PIL image
        if not isinstance(image, np.ndarray):
            raise TypeError(f"Unsupported image type {type(image)}")
        if image.dtype != np.uint8:
            raise ValueError("Image type has to be uint8")
        if image.ndim != 3 or image.shape[2] != 3:
            raise ValueError(f"Invalid shape for rgb image: {image.shape}")
        image = resizer(image, self.max_resolution)
        mode, as_jpg = self.choose_mode(image)
        destination['mode'] = IMAGE_MODES[mode] if mode in IMAGE_MODES else -1
        destination['height'], destination['width'] = image.shape[:2]
        if mode == 'jpg':
            if as_jpg is None:
                as_jpg = self.encode_jpeg(image)
            destination['data_ptr'], storage = malloc(as_jpg.nbytes)
            storage[:] = as_jpg
        elif mode == 'raw':
            flat = np.ascontiguousarray(image).view('<u1').reshape(-1)
            destination['data_ptr'], storage = malloc(image.nbytes)
            storage[:] = flat
        else:
            raise ValueError(f"Unsupported write mode {self.write_mode}")
