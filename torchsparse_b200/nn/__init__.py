from . import functional
from .modules import *
from .fused import *
