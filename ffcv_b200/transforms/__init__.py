from .color_jitter import RandomBrightness, RandomContrast, RandomSaturation
from .common import Squeeze
from .cutout import Cutout
from .flip import RandomHorizontalFlip
from .mixup import ImageMixup, LabelMixup, MixupToOneHot
from .module import ModuleWrapper
from .normalize import NormalizeImage
from .ops import Convert, ToDevice, ToTensor, ToTorchImage, View
from .poisoning import Poison
from .random_resized_crop import RandomResizedCrop
from .replace_label import ReplaceLabel
from .translate import RandomTranslate

__all__ = ['ToTensor', 'ToDevice', 'ToTorchImage', 'NormalizeImage', 'Convert', 'View', 'Squeeze',
           'Cutout', 'RandomHorizontalFlip', 'RandomTranslate', 'RandomResizedCrop', 'ModuleWrapper',
           'RandomBrightness', 'RandomContrast', 'RandomSaturation', 'ImageMixup', 'LabelMixup',
           'MixupToOneHot', 'Poison', 'ReplaceLabel']
