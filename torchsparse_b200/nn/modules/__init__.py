from .activation import *
from .conv import *
from .norm import *
from .tensor_ops import *
