"""tilekernels_b200 -- B200 (sm_100a) implementation of the TileKernels quantization casts.

`tilekernels_b200.quant` exposes the entry points of the reference's `tile_kernels.quant`
hot path under the same names, argument lists and return conventions.  Every call
ends in one hand-written CUDA kernel of libtkquant.so (C ABI, see include/tkquant.h);
there is no other backend and no CPU path: importing `quant` without the built
library raises.
"""
from . import config, utils  # noqa: F401
from . import quant  # noqa: F401
from . import testing  # noqa: F401

__version__ = '0.1.0'
