"""swiglu_forward_and_per_channel_cast_and_transpose
(reference: tile_kernels/quant/swiglu_forward_and_per_channel_cast_and_transpose_kernel.py:177-231)."""
from typing import Optional

import torch

from .. import _lib
from .common import current_stream_ptr, device_guard
from .types import QuantTensor


def swiglu_forward_and_per_channel_cast_and_transpose(
    x: torch.Tensor,
    fmt: str,
    num_per_tokens: int,
    round_sf: bool = False,
    without_transpose: bool = False,
    swiglu_clamp_value: Optional[float] = None,
) -> QuantTensor:
    """silu(x[:, :hidden]) * x[:, hidden:] rounded to bfloat16, then FP8 e4m3 with one scale per
    (num_per_tokens tokens x 1 channel); the data are written transposed unless `without_transpose`.

    Args:
        x: contiguous CUDA bfloat16 tensor (num_tokens, 2 * hidden); num_tokens % 128 == 0.
        num_per_tokens: 32 or 128.

    Returns:
        (out, out_sf): float8_e4m3fn (hidden, num_tokens) [or (num_tokens, hidden)] and float32
        (num_tokens / num_per_tokens, hidden).
    """
    assert fmt == 'e4m3'
    assert x.dim() == 2 and x.is_contiguous() and x.is_cuda
    assert x.dtype == torch.bfloat16
    num_tokens, hidden = x.shape
    assert num_tokens % 128 == 0 and hidden % 128 == 0
    assert num_per_tokens in (32, 128)
    hidden = hidden // 2

    out = torch.empty((num_tokens, hidden) if without_transpose else (hidden, num_tokens), dtype=torch.float8_e4m3fn, device=x.device)
    out_sf = torch.empty((num_tokens // num_per_tokens, hidden), dtype=torch.float32, device=x.device)
    if num_tokens > 0:
        with device_guard(x.device):
            rc = _lib.lib().tkq_swiglu_forward_and_per_channel_cast(
                x.data_ptr(), num_tokens, hidden, num_per_tokens, 0 if without_transpose else 1,
                -1.0 if swiglu_clamp_value is None else float(swiglu_clamp_value), _lib.ROUND_SF if round_sf else 0,
                out.data_ptr(), out_sf.data_ptr(), current_stream_ptr(x.device))
        _lib.check(rc, 'tkq_swiglu_forward_and_per_channel_cast')
    return out, out_sf
