from .base import Field
from .basics import FloatField, IntField
from .ndarray import NDArrayField, TorchTensorField
from .rgb_image import RGBImageField

__all__ = ['Field', 'FloatField', 'IntField', 'NDArrayField', 'RGBImageField', 'TorchTensorField']
