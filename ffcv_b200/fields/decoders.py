from .basics import FloatDecoder, IntDecoder
from .rgb_image import (CenterCropRGBImageDecoder, RandomResizedCropRGBImageDecoder,
                        SimpleRGBImageDecoder)

__all__ = ['FloatDecoder', 'IntDecoder', 'CenterCropRGBImageDecoder',
           'RandomResizedCropRGBImageDecoder', 'SimpleRGBImageDecoder']
