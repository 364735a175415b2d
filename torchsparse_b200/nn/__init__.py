from . import functional
from .modules import *
