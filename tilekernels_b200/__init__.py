"""tilekernels_b200 -- B200 (sm_100a) implementation of the TileKernels quantization casts.

`tilekernels_b200.quant` exposes the entry points of the reference's `tile_kernels.quant`
hot path under the same names, argument lists and return conventions.  Every call
ends in one hand-written CUDA kernel of libtkquant.so (C ABI, see include/tkquant.h);
there is no other backend and no CPU path: importing `quant` without the built
library raises.

Sub-modules load on first use, so that `python -m tilekernels_b200.build` can run before
the library exists.
"""
import importlib

__version__ = '0.1.0'
_SUBMODULES = ('config', 'utils', 'quant', 'moe', 'testing', 'host', 'sharding', 'build')


def __getattr__(name):
    if name in _SUBMODULES:
        return importlib.import_module(f'{__name__}.{name}')
    raise AttributeError(f'module {__name__!r} has no attribute {name!r}')
