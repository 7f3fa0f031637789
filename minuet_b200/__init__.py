"""minuet_b200: the Minuet sparse-convolution hot path rebuilt for B200 (sm_100a).

Same Python surface as ``minuet`` for that path: ``SparseTensor``,
``nn.SparseConv3d`` / ``nn.SparseConv`` / ``nn.KernelMapCache``,
``nn.functional.*`` and the helpers ``set_kernel_map_cache``, ``autotune``,
``load_tunable_config`` and ``dump_tunable_config``.
"""
from .tensors import *
from . import nn
from . import utils
from .nn.functional.convolution import set_gemm_parallel_level
from .utils.helpers import set_kernel_map_cache
from .utils.helpers import autotune
from .utils.helpers import load_tunable_config
from .utils.helpers import dump_tunable_config
