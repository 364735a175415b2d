from .blocks import *
from .resnet import *
from .unet import *
