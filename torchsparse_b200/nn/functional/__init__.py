from .conv import *
from .count import *
from .devoxelize import *
from .hash import *
from .query import *
from .voxelize import *
from .tensor_ops import *
