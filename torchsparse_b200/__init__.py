"""torchsparse_b200: the sparse-convolution hot path of TorchSparse, rebuilt for B200 (sm_100a).

Python surface as in the reference (``SparseTensor``, ``nn.Conv3d``, ``nn.functional.conv3d``
with the ImplicitGEMM / GatherScatter / FetchOnDemand dataflows, ``sparse_quantize``, the
backbones); every native operator goes through the tsb200 C ABI (include/tsb200.h)."""
from . import backends
from . import backend  # loads libtsb200.so; raises ImportError when it has not been built
from .operators import *
from .tensor import *
from .version import __version__

backends.init()
