"""The one MoE entry point next to the quantization path: row expansion with scale factors
(reference: tile_kernels/moe/__init__.py, expand_to_fused_kernel.py).  The rest of the reference's moe package
(gating, mapping, reduction) is outside this library."""
from .. import _lib as _lib_module

_lib_module.lib()  # fail at import when the CUDA library is missing

from .expand_to_fused_kernel import expand_to_fused, expand_to_fused_with_sf  # noqa: E402
