"""Scale-factor geometry and cast configuration shared by the quant entry points.

Mirrors the host-side part of the reference's tile_kernels/quant/common.py: the
config records (:20-59), input/output config construction (:62-113), the
scale-factor shapes, allocation and epilogue (:130-193) and the FP4 unpacker
(:247-295).  The device-side macros of that file (get_sf_and_inv, load_sf,
store_sf) live in csrc/tkq_common.cuh.
"""
import contextlib
from dataclasses import dataclass, replace
from typing import Optional, Union

import torch

from .. import _lib
from ..utils import align, ceil_div
from .types import QuantTensor

_FMT_TO_DTYPE = {'e5m6': torch.uint32, 'e4m3': torch.float8_e4m3fn, 'e2m1': torch.int8}
FMT_TO_ENUM = {'e4m3': _lib.FMT_E4M3, 'e2m1': _lib.FMT_E2M1, 'e5m6': _lib.FMT_E5M6}
DTYPE_TO_ENUM = {torch.bfloat16: _lib.DT_BF16, torch.float32: _lib.DT_FP32}


@dataclass(frozen=True)
class BaseCastConfig:
    torch_dtype: torch.dtype = torch.float8_e4m3fn
    sf_block: tuple[int, int] = (1, 1)
    use_tma_aligned_col_major_sf: bool = False
    use_packed_ue8m0: bool = False

    @property
    def sf_torch_dtype(self) -> torch.dtype:
        return torch.uint8 if self.use_packed_ue8m0 else torch.float32


@dataclass(frozen=True)
class CastInputConfig(BaseCastConfig):
    with_sf: bool = True

    @property
    def flags(self) -> int:
        """Layout bits of include/tkquant.h for the scales of an already quantized input."""
        return (_lib.SF_COL_MAJOR if self.use_tma_aligned_col_major_sf else 0) | (_lib.SF_UE8M0 if self.use_packed_ue8m0 else 0)


@dataclass(frozen=True)
class CastOutputConfig(BaseCastConfig):
    round_sf: bool = False
    custom_clamp_min_value: Optional[float] = None

    @property
    def clamp_min_value(self) -> float:
        if self.custom_clamp_min_value is not None:
            return self.custom_clamp_min_value
        if self.torch_dtype == torch.float8_e4m3fn:
            return 1e-4
        if self.torch_dtype == torch.int8:
            return 6.0 * 2.0 ** -126
        raise ValueError(f'Unsupported dtype {self.torch_dtype}')

    @property
    def flags(self) -> int:
        """Flag bits of include/tkquant.h for this output layout."""
        f = 0
        if self.round_sf:
            f |= _lib.ROUND_SF
        if self.use_tma_aligned_col_major_sf:
            f |= _lib.SF_COL_MAJOR
        if self.use_packed_ue8m0:
            f |= _lib.SF_UE8M0
        return f


def get_cast_input_and_config(
    x: Union[torch.Tensor, QuantTensor],
    sf_block: Optional[tuple[int, int]],
) -> tuple[torch.Tensor, Optional[torch.Tensor], CastInputConfig]:
    """Normalise the input of a cast.  A plain tensor must be bfloat16 / float32.  A `(data, scales)` pair is an
    already quantized tensor: its scale layout is recognised from strides and dtype (unit stride along tokens =
    column-major; int32 = packed ue8m0) and the scales come back as their row-major *storage* (a transposed view,
    bytes for the packed layout), as in the reference (tile_kernels/quant/common.py:62-88)."""
    if isinstance(x, tuple):
        assert isinstance(sf_block, tuple)
        x, x_sf = x
        config = CastInputConfig(torch_dtype=x.dtype, with_sf=True, sf_block=tuple(sf_block))
        assert isinstance(x, torch.Tensor) and isinstance(x_sf, torch.Tensor)
        assert x.dtype in (torch.float8_e4m3fn, torch.int8, torch.uint8)
        if x_sf.stride(0) == 1:
            config = replace(config, use_tma_aligned_col_major_sf=True)
            x_sf = x_sf.T
            if x_sf.dtype == torch.int32:
                config = replace(config, use_packed_ue8m0=True)
                x_sf = x_sf.view(torch.uint8)
        else:
            assert x_sf.stride(1) == 1
            assert x_sf.dtype == torch.float32
        return x, x_sf, config
    assert sf_block is None
    assert isinstance(x, torch.Tensor)
    assert x.dtype in (torch.bfloat16, torch.float32)
    return x, None, CastInputConfig(torch_dtype=x.dtype, with_sf=False)


def get_cast_output_config(
    fmt: str,
    sf_block: tuple[int, int],
    use_tma_aligned_col_major_sf: bool = False,
    round_sf: bool = False,
    use_packed_ue8m0: bool = False,
    custom_clamp_min_value: Optional[float] = None,
) -> CastOutputConfig:
    assert fmt in ('e5m6', 'e4m3', 'e2m1')
    # Packed exponent bytes only exist in the column-major layout (the reference's store
    # macro addresses them that way regardless of the flag, tile_kernels/quant/common.py:238-240).
    assert use_tma_aligned_col_major_sf or not use_packed_ue8m0, 'use_packed_ue8m0 needs use_tma_aligned_col_major_sf'
    return CastOutputConfig(
        torch_dtype=_FMT_TO_DTYPE[fmt],
        sf_block=sf_block,
        use_tma_aligned_col_major_sf=use_tma_aligned_col_major_sf,
        round_sf=round_sf,
        use_packed_ue8m0=use_packed_ue8m0,
        custom_clamp_min_value=custom_clamp_min_value,
    )


def get_logical_hidden(hidden: int, dtype: torch.dtype) -> int:
    """Number of values in a row whose storage dtype packs two FP4 per int8."""
    return hidden * 2 if dtype == torch.int8 else hidden


def get_physical_hidden(hidden: int, dtype: torch.dtype) -> int:
    """Number of storage elements for `hidden` values (two FP4 per int8)."""
    return hidden // 2 if dtype == torch.int8 else hidden


def get_sf_shape(shape: tuple[int, int], config: BaseCastConfig) -> tuple[int, int]:
    """Storage shape of the scale tensor before alignment padding.

    Row-major: (token blocks, channel blocks).  Column-major: transposed.  Packed
    ue8m0 (uint8 storage): (ceil(channel blocks / 4), 4 * token blocks)."""
    blocks_m = ceil_div(shape[0], config.sf_block[0])
    blocks_k = ceil_div(shape[1], config.sf_block[1])
    if config.use_packed_ue8m0:
        blocks_m, blocks_k = blocks_m * 4, ceil_div(blocks_k, 4)
    return (blocks_k, blocks_m) if config.use_tma_aligned_col_major_sf else (blocks_m, blocks_k)


def alloc_scaling_factors(shape: tuple[int, int], out_config: BaseCastConfig,
                          device: Union[torch.device, str] = 'cuda') -> torch.Tensor:
    """Allocate scale storage; column-major rows are padded to 16 bytes (4 fp32 or 16 exponent bytes)
    and the returned tensor is the unpadded slice of that storage."""
    rows, cols = get_sf_shape(shape, out_config)
    pitch = cols
    if out_config.use_tma_aligned_col_major_sf:
        pitch = align(cols, 16 if out_config.use_packed_ue8m0 else 4)
    storage = torch.empty((rows, pitch), dtype=out_config.sf_torch_dtype, device=device)
    return storage[:, :cols] if out_config.use_tma_aligned_col_major_sf else storage


def cast_epilogue(out_sf: torch.Tensor, num_tokens: int, hidden: int, config: BaseCastConfig) -> torch.Tensor:
    """Storage -> the tensor handed to the caller: exponent bytes viewed as int32 words,
    column-major storage transposed back to (token blocks, channel blocks)."""
    if config.use_packed_ue8m0:
        if num_tokens == 0:
            out_sf = torch.empty((out_sf.shape[0], out_sf.shape[1] // 4), dtype=torch.int32, device=out_sf.device)
        else:
            out_sf = out_sf.view(dtype=torch.int32)
    if config.use_tma_aligned_col_major_sf:
        out_sf = out_sf.T
    return out_sf[:ceil_div(num_tokens, config.sf_block[0]), :]


def sf_stride_for_kernel(out_sf: torch.Tensor) -> int:
    """The `sf_stride` argument of the C ABI: elements between consecutive storage rows."""
    return out_sf.stride(0)


def current_stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


_NO_GUARD = contextlib.nullcontext()


def device_guard(device: torch.device):
    """Context that makes `device` current for the C call.  Switching and restoring the device costs several
    microseconds per call, more than a third of a small cast's wrapper time: nothing is switched when `device` is
    current already, which is the usual case."""
    return _NO_GUARD if device.index == torch.cuda.current_device() else torch.cuda.device(device)


_E2M1_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0)


def unpack_from_e2m1fn_x2(x: torch.Tensor, out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """Decode packed FP4 (two e2m1 codes per byte, even index in the low nibble) to `out_dtype`;
    the last dimension doubles.  Debugging helper, plain torch."""
    assert x.dtype in (torch.int8, torch.uint8)
    if x.ndim == 0:
        raise ValueError('x must have at least 1 dimension so the last dim can be doubled')
    table = torch.tensor(_E2M1_VALUES, dtype=torch.float32, device=x.device)
    codes = x.view(torch.uint8).to(torch.int64)
    pairs = torch.stack([codes & 0xF, codes >> 4], dim=-1)
    return table[pairs].reshape(*x.shape[:-1], x.shape[-1] * 2).to(out_dtype)
