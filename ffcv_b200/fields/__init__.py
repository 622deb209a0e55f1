from .base import Field
from .basics import FloatField, IntField
from .rgb_image import RGBImageField

__all__ = ['Field', 'FloatField', 'IntField', 'RGBImageField']
