from . import functional
from .convolutions import *
from .activations import *
from .normalizations import *
from .pooling import *
