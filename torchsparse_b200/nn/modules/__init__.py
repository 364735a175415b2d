from .activation import *
from .conv import *
from .norm import *
from .crop import *
from .pooling import *
