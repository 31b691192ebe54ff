"""per_channel_cast_fused (reference: tile_kernels/quant/per_channel_cast_fused_kernel.py:137-203).

Implemented: the plain bfloat16 / float32 input.  The FP8-input rescale and the
`pos_to_token` gather of the reference are not implemented yet and raise."""
from typing import Optional, Union

import torch

from .. import _lib
from ..utils import ceil_div
from .common import DTYPE_TO_ENUM, current_stream_ptr
from .types import QuantTensor


def per_channel_cast_fused(
    x: Union[torch.Tensor, QuantTensor],
    fmt: str,
    num_per_tokens: int,
    round_sf: bool = False,
    num_per_channels: Optional[int] = None,
    pos_to_token: Optional[torch.Tensor] = None,
) -> QuantTensor:
    """Cast a matrix to FP8 e4m3 with one scale per (128 tokens x 1 channel)."""
    if isinstance(x, tuple) or num_per_channels is not None or pos_to_token is not None:
        raise NotImplementedError('per_channel_cast_fused: FP8 inputs and pos_to_token are not implemented in tilekernels_b200 yet')
    assert fmt == 'e4m3'
    assert x.dim() == 2 and x.is_contiguous() and x.is_cuda
    assert x.dtype in (torch.bfloat16, torch.float32)
    num_tokens, hidden = x.shape
    assert num_tokens % 128 == 0
    assert hidden % 64 == 0
    assert num_per_tokens == 128

    out = torch.empty((num_tokens, hidden), dtype=torch.float8_e4m3fn, device=x.device)
    out_sf = torch.empty((ceil_div(num_tokens, num_per_tokens), hidden), dtype=torch.float32, device=x.device)
    if num_tokens > 0:
        with torch.cuda.device(x.device):
            rc = _lib.lib().tkq_per_channel_cast(
                x.data_ptr(), DTYPE_TO_ENUM[x.dtype], num_tokens, hidden, _lib.ROUND_SF if round_sf else 0, out.data_ptr(),
                out_sf.data_ptr(), current_stream_ptr(x.device))
        _lib.check(rc, 'tkq_per_channel_cast')
    return out, out_sf
