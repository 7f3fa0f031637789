from .indexing import *
from .hash import *
from .scan import *
from .convolution import *
from .memory import *
from .pooling import *
from .concat import *
from .voxelize import *
