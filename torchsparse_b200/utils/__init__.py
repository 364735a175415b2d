from .utils import *
from .tensor_cache import *
from .to_dense import *
from .quantize import *
