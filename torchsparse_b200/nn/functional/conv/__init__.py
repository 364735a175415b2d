from .conv import *
from .conv_mode import *
from . import conv_config
from .conv_config import Dataflow, ConvConfig
from .kmap import *
from .downsample import *
from .func import *
