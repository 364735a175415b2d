from .activation import *
from .bev import *
from .conv import *
from .norm import *
from .tensor_ops import *
