from .common import Squeeze
from .cutout import Cutout
from .flip import RandomHorizontalFlip
from .module import ModuleWrapper
from .normalize import NormalizeImage
from .ops import Convert, ToDevice, ToTensor, ToTorchImage, View
from .random_resized_crop import RandomResizedCrop
from .translate import RandomTranslate

__all__ = ['ToTensor', 'ToDevice', 'ToTorchImage', 'NormalizeImage', 'Convert', 'View', 'Squeeze',
           'Cutout', 'RandomHorizontalFlip', 'RandomTranslate', 'RandomResizedCrop', 'ModuleWrapper']
