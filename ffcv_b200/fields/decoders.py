from .basics import FloatDecoder, IntDecoder
from .ndarray import NDArrayDecoder
from .rgb_image import (CenterCropRGBImageDecoder, RandomResizedCropRGBImageDecoder,
                        SimpleRGBImageDecoder)

__all__ = ['FloatDecoder', 'IntDecoder', 'NDArrayDecoder', 'CenterCropRGBImageDecoder',
           'RandomResizedCropRGBImageDecoder', 'SimpleRGBImageDecoder']
