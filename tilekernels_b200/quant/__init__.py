"""Quantization entry points, named as in the reference's tile_kernels/quant/__init__.py:1-11."""
from .. import _lib as _lib_module

_lib_module.lib()  # fail at import, not at first call, when the CUDA library is missing

from .cast_back_e5m6_kernel import cast_back_e5m6  # noqa: E402
from .cast_back_kernel import cast_back, per_token_cast_back  # noqa: E402
from .common import unpack_from_e2m1fn_x2  # noqa: E402
from .per_block_cast_lossless_kernel import per_block_cast_lossless  # noqa: E402
from .per_block_cast_kernel import per_block_cast, per_block_cast_with_precomputed_sf, per_block_cast_with_sf_only  # noqa: E402
from .per_channel_cast_and_transpose_kernel import per_channel_cast_and_transpose  # noqa: E402
from .per_channel_cast_fused_kernel import per_channel_cast_fused  # noqa: E402
from .per_channel_cast_kernel import per_channel_cast  # noqa: E402
from .per_token_cast_kernel import per_token_cast, per_token_cast_with_precomputed_sf, per_token_cast_with_sf_only  # noqa: E402
from .per_token_cast_to_e5m6_kernel import per_token_cast_to_e5m6  # noqa: E402
from .swiglu_backward_and_per_token_cast_kernel import swiglu_backward_and_per_token_cast  # noqa: E402
from .swiglu_forward_and_per_channel_cast_and_transpose_kernel import swiglu_forward_and_per_channel_cast_and_transpose  # noqa: E402
from .swiglu_forward_and_per_token_cast_kernel import swiglu_forward_and_per_token_cast  # noqa: E402
from .types import QuantTensor  # noqa: E402
