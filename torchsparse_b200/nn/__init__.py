from . import functional
from .modules import *
from .fused import *
from .static_engine import *
