"""CPU oracle for the quantization casts -- TEST INFRASTRUCTURE ONLY.

Only tests/, the smoke check and the CPU-baseline legs of bench.py import this
package; tilekernels_b200 never does.  The arithmetic lives in tkq_oracle.c
(a restatement of the reference's tile_kernels/torch/{cast,cast_e5m6,swiglu}.py,
cited function by function there).  This wrapper hands torch CPU tensors to it
and lays the scale factors out the way the reference returns them
(tile_kernels/torch/cast.py:199-219, cast_e5m6.py:23-34,190-216), so that a
test can compare dtype, shape, strides and bytes.
"""
import ctypes
import os
from typing import Optional

import numpy as np
import torch

from .build import LIB, build as build_library

_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB):
            build_library()
        _lib = ctypes.CDLL(LIB)
        _lib.tkq_expf.restype = ctypes.c_float
        _lib.tkq_expf.argtypes = [ctypes.c_float]
    return _lib


def _ceil_div(a: int, b: int) -> int:
    return (a + b - 1) // b


def _align(a: int, b: int) -> int:
    return _ceil_div(a, b) * b


_DT = {torch.bfloat16: 0, torch.float32: 1}
_FMT = {'e4m3': 0, 'e2m1': 1}
_vp = ctypes.c_void_p
_i64 = ctypes.c_int64


def _rows(x: torch.Tensor):
    assert x.device.type == 'cpu' and x.dim() == 2 and x.dtype in _DT
    if x.shape[1] > 0 and x.stride(1) != 1:
        x = x.contiguous()
    return x


def format_sf(bits: torch.Tensor, col_major: bool, packed_ue8m0: bool) -> torch.Tensor:
    """Row-major int32 scale bits [nm, nk] -> the reference's returned scale tensor.

    row-major:   fp32 [nm, nk]
    col-major:   fp32 [nm, nk] with strides (1, align(nm, 4)), padding zero
    packed:      int32 [nm, ceil(nk/4)] with strides (1, align(nm, 4)); byte b of
                 word k is the exponent byte of group 4k+b, padding zero
    (tile_kernels/torch/cast.py:199-219)
    """
    nm, nk = bits.shape
    if not col_major:
        return bits.view(torch.float32)
    nm_pad = _align(nm, 4)
    if packed_ue8m0:
        nkw = _ceil_div(nk, 4)
        exp_bytes = torch.zeros((nm, nkw * 4), dtype=torch.uint8)
        exp_bytes[:, :nk] = (bits >> 23).to(torch.uint8)
        words = exp_bytes.view(torch.int32)  # [nm, nkw]
        storage = torch.zeros((nkw, nm_pad), dtype=torch.int32)
        storage[:, :nm] = words.T
        return storage.T[:nm, :]
    storage = torch.zeros((nk, nm_pad), dtype=torch.float32)
    storage[:, :nm] = bits.view(torch.float32).T
    return storage.T[:nm, :]


def cast(x: torch.Tensor, fmt: str, block_size=(32, 32), sf: Optional[torch.Tensor] = None, round_sf: bool = False,
         use_tma_aligned_col_major_sf: bool = False, use_packed_ue8m0: bool = False,
         clamp_min: Optional[float] = None, x_block_size=None):
    """Same contract as the reference's tile_kernels.torch.cast (cast.py:62-221).  An already quantized input
    `(data, scales)` with `x_block_size` is dequantised to fp32 first (data * scale, cast.py:86-97) and then
    cast like any fp32 tensor.  Returns `out` when `sf` is given, else `(out, out_sf)`."""
    if isinstance(x, tuple):
        assert x_block_size is not None
        x = cast_back(x, 'fp32', x_block_size)
    x = _rows(x)
    T, H = x.shape
    bm, bk = block_size
    is_fp4 = fmt == 'e2m1'
    out_dtype = torch.int8 if is_fp4 else torch.float8_e4m3fn
    out = torch.empty((T, H // 2 if is_fp4 else H), dtype=torch.uint8)
    nm, nk = _ceil_div(T, bm), _ceil_div(H, bk)
    bits = torch.zeros((nm, nk), dtype=torch.int32)
    sf_ptr = None
    if sf is not None:
        assert not use_packed_ue8m0 and not use_tma_aligned_col_major_sf
        assert tuple(sf.shape) == (nm, nk) and sf.dtype == torch.float32
        sf_c = sf.contiguous()
        sf_ptr = _vp(sf_c.data_ptr())
    if T > 0:
        rc = lib().tkqo_cast(_vp(x.data_ptr()), _DT[x.dtype], _i64(T), _i64(H), _i64(x.stride(0)), _FMT[fmt],
                             int(bm), int(bk), int(round_sf),
                             ctypes.c_float(-1.0 if clamp_min is None else clamp_min), sf_ptr,
                             _vp(out.data_ptr()), _vp(bits.data_ptr()))
        assert rc == 0, f'oracle cast failed ({rc})'
    out = out.view(out_dtype)
    if sf is not None:
        return out
    if T == 0:  # shapes of the empty case, cast.py:109-123
        if use_packed_ue8m0:
            return out, torch.empty((_ceil_div(nk, 4), 0), dtype=torch.int32).T
        if use_tma_aligned_col_major_sf:
            return out, torch.empty((nk, 0), dtype=torch.float32).T
        return out, torch.empty((0, nk), dtype=torch.float32)
    return out, format_sf(bits, use_tma_aligned_col_major_sf, use_packed_ue8m0)


def cast_back(x, fmt: str, block_size=(32, 32)) -> torch.Tensor:
    """Dequantise (q, sf) to fp32 or bf16 (tile_kernels/torch/cast.py:40-59)."""
    q, sf = x
    is_fp4 = q.dtype == torch.int8
    T = q.shape[0]
    H = q.shape[1] * (2 if is_fp4 else 1)
    bm, bk = block_size
    sf32 = sf_to_float(sf)[:, :_ceil_div(H, bk)].contiguous()
    out = torch.empty((T, H), dtype=torch.float32)
    if T > 0:
        lib().tkqo_cast_back(_vp(q.contiguous().data_ptr()), 1 if is_fp4 else 0, _i64(T), _i64(H), int(bm), int(bk),
                             _vp(sf32.data_ptr()), _vp(out.data_ptr()))
    return out if fmt == 'fp32' else out.bfloat16()


def cast_back_from_e5m6(x, fmt: str, x_block_size) -> torch.Tensor:
    """Dequantise packed E5M6 (tile_kernels/torch/cast_e5m6.py:221-258)."""
    data, sf = x
    assert data.dtype == torch.uint8
    T = data.shape[0]
    H = data.shape[1] * 2 // 3
    bm, bk = x_block_size
    sf32 = sf_to_float(sf)[:, :_ceil_div(H, bk)].contiguous()
    out = torch.empty((T, H), dtype=torch.float32)
    if T > 0:
        rc = lib().tkqo_cast_back_e5m6(_vp(data.contiguous().data_ptr()), _i64(T), _i64(H), int(bm), int(bk), _vp(sf32.data_ptr()),
                                       _vp(out.data_ptr()))
        assert rc == 0
    return out if fmt == 'fp32' else out.bfloat16()


def per_block_cast_lossless(x, x_block_size, out_block_size, use_tma_aligned_col_major_sf: bool = False,
                            use_packed_ue8m0: bool = False):
    """Restatement of the reference kernel tile_kernels/quant/per_block_cast_lossless_kernel.py:96-131 (it has no
    PyTorch counterpart; its test checks that both sides dequantise to the same fp32 values): output exponent =
    max input exponent in the block - 6, not below 0; value = fp4 * 2^(e_in - e_out) cast to e4m3."""
    q, sf = x
    T = q.shape[0]
    H = q.shape[1] * 2
    ibm, ibk = x_block_size
    obm, obk = out_block_size
    e_in = (sf_to_float(sf)[:, :_ceil_div(H, ibk)].contiguous().view(torch.int32) >> 23)  # [T/ibm, H/ibk]
    e_elem = e_in.repeat_interleave(ibm, 0)[:T].repeat_interleave(ibk, 1)[:, :H]
    nm, nk = _ceil_div(T, obm), _ceil_div(H, obk)
    padded = torch.zeros((nm * obm, nk * obk), dtype=torch.int32)
    padded[:T, :H] = e_elem
    e_out = padded.view(nm, obm, nk, obk).amax(dim=(1, 3))
    e_out = torch.where(e_out >= 6, e_out - 6, torch.zeros_like(e_out))
    e_out_elem = e_out.repeat_interleave(obm, 0)[:T].repeat_interleave(obk, 1)[:, :H]
    rel = ((e_elem - e_out_elem + 127) << 23).view(torch.float32)
    fp4 = cast_back((q, torch.ones((T, H // 32), dtype=torch.float32)), 'fp32', (1, 32))  # the bare e2m1 values
    out = (fp4 * rel).clamp(-448, 448).to(torch.float8_e4m3fn)
    return out, format_sf((e_out << 23).contiguous(), use_tma_aligned_col_major_sf, use_packed_ue8m0)


def sf_to_float(sf: torch.Tensor) -> torch.Tensor:
    """fp32 scales unchanged; packed int32 ue8m0 words -> fp32 [nm, 4*words] (cast.py:28-37)."""
    if sf.dtype == torch.float32:
        return sf
    assert sf.dtype == torch.int32
    dense = torch.empty(sf.shape, dtype=sf.dtype)
    dense.copy_(sf)
    b = dense.view(torch.uint8).to(torch.int32)
    return (b << 23).view(torch.float32)


def per_channel_cast_fused(x, num_per_tokens: int, num_per_channels: Optional[int], round_sf: bool,
                           pos_to_token: Optional[torch.Tensor]):
    """Same contract as tile_kernels.torch.per_channel_cast_fused (per_channel_cast_fused.py:9-44): gather rows
    through pos_to_token (negative = a row of zeros, data and scales), then the (128, 1)-block cast; FP8 input
    carries one scale per (token, num_per_channels) that is multiplied in first."""
    fused = isinstance(x, tuple)
    if pos_to_token is not None:
        idx = pos_to_token.clamp(min=0).long()
        valid = (pos_to_token >= 0).unsqueeze(1)
        data = x[0] if fused else x
        gathered = torch.where(valid, data[idx].float(), torch.zeros(())).to(data.dtype)
        x = (gathered, torch.where(valid, x[1][idx], torch.zeros(()))) if fused else gathered
    return cast(x, 'e4m3', (num_per_tokens, 1), round_sf=round_sf, x_block_size=(1, num_per_channels) if fused else None)


def cast_to_e5m6(x: torch.Tensor, num_per_channels: int, use_tma_aligned_col_major_sf: bool = False,
                 round_sf: bool = False, use_packed_ue8m0: bool = False):
    """Same contract as tile_kernels.torch.cast_to_e5m6 (cast_e5m6.py:135-218)."""
    x = _rows(x)
    T, H = x.shape
    g = num_per_channels
    assert H % g == 0 and H % 8 == 0 and g % 8 == 0
    ng = H // g
    words = torch.empty((T, H // 8 * 3), dtype=torch.int32)
    sfw = torch.zeros((T, ng), dtype=torch.int32)
    if T > 0:
        rc = lib().tkqo_cast_e5m6(_vp(x.data_ptr()), _DT[x.dtype], _i64(T), _i64(H), _i64(x.stride(0)), _i64(g),
                                  int(round_sf), int(use_packed_ue8m0), _vp(words.data_ptr()), _vp(sfw.data_ptr()))
        assert rc == 0
    packed = words.view(torch.uint8)
    if use_packed_ue8m0:
        ngw = _ceil_div(ng, 4)
        eb = torch.zeros((T, ngw * 4), dtype=torch.uint8)
        eb[:, :ng] = sfw.to(torch.uint8)
        sf_out = eb.view(torch.int32)
    else:
        sf_out = sfw.view(torch.float32)
    if use_tma_aligned_col_major_sf:  # cast_e5m6.py:23-34
        storage = torch.zeros((sf_out.shape[1], _align(T, 4)), dtype=sf_out.dtype)
        storage[:, :T] = sf_out.T
        sf_out = storage.T[:T, :]
    return packed, sf_out


def swiglu_forward(x: torch.Tensor, pos_to_token_topk: Optional[torch.Tensor] = None,
                   topk_weights: Optional[torch.Tensor] = None, swiglu_clamp_value: Optional[float] = None,
                   clamped_count: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Same contract as tile_kernels.torch.swiglu_forward (swiglu.py:9-88); exp() is tkq_expf."""
    assert x.dim() == 2 and x.is_contiguous() and x.dtype in _DT
    T, H2 = x.shape
    H = H2 // 2
    y = torch.empty((T, H), dtype=torch.float32)
    pos_ptr = w_ptr = cnt_ptr = None
    if pos_to_token_topk is not None:
        pos = pos_to_token_topk.to(torch.int32).contiguous()
        w = topk_weights.to(torch.float32).contiguous()
        pos_ptr, w_ptr = _vp(pos.data_ptr()), _vp(w.data_ptr())
    if clamped_count is not None:
        assert clamped_count.dtype == torch.int64 and clamped_count.is_contiguous()
        cnt_ptr = _vp(clamped_count.data_ptr())
    if T > 0:
        lib().tkqo_swiglu_forward(_vp(x.data_ptr()), _DT[x.dtype], _i64(T), _i64(H),
                                  ctypes.c_float(-1.0 if swiglu_clamp_value is None else swiglu_clamp_value),
                                  cnt_ptr, pos_ptr, w_ptr, _vp(y.data_ptr()))
    return y


def swiglu_backward(x, grad_out: torch.Tensor, weight: torch.Tensor, pos_to_token_topk: torch.Tensor,
                    token_topk_to_pos: torch.Tensor, num_per_channels: int,
                    swiglu_clamp_value: Optional[float] = None):
    """Same contract as tile_kernels.torch.swiglu_backward (swiglu.py:98-226): returns fp32 (out, x_grad_full,
    weight_grad).  exp() is tkq_expf; the row sums of weight_grad are accumulated in double."""
    assert num_per_channels in (32, 128)
    data, _ = x
    assert data.shape[-1] % (2 * num_per_channels) == 0
    H = data.shape[-1] // 2
    xf = cast_back((data.view(-1, 2 * H), x[1]), 'fp32', (1, num_per_channels)).contiguous()
    T = xf.shape[0]
    g = grad_out.view(-1, H).contiguous()
    assert g.dtype == torch.bfloat16 and g.shape == (T, H)
    w = weight.to(torch.float32).contiguous()
    assert w.shape == token_topk_to_pos.shape
    pos = pos_to_token_topk.to(torch.int32).contiguous()
    out = torch.empty((T, H), dtype=torch.float32)
    x_grad = torch.empty((T, 2 * H), dtype=torch.float32)
    weight_grad = torch.zeros_like(w)
    if T > 0:
        lib().tkqo_swiglu_backward(_vp(xf.data_ptr()), _vp(g.data_ptr()), _i64(T), _i64(H),
                                   ctypes.c_float(-1.0 if swiglu_clamp_value is None else swiglu_clamp_value),
                                   _vp(pos.data_ptr()), _vp(w.data_ptr()), _vp(out.data_ptr()), _vp(x_grad.data_ptr()),
                                   _vp(weight_grad.data_ptr()))
    return out, x_grad, weight_grad


def expand_to_fused(x: torch.Tensor, token_topk_to_pos: torch.Tensor, pos_to_expert: torch.Tensor) -> torch.Tensor:
    """Row expansion (tile_kernels/torch/expand_to_fused.py:6-39): token t goes to every position
    token_topk_to_pos[t, k] >= 0, every other row of the result is zero."""
    num_expanded = pos_to_expert.shape[0]
    dense = torch.empty(x.shape, dtype=x.dtype)
    dense.copy_(x)
    rows = dense.view(torch.uint8).numpy().reshape(x.shape[0], -1)
    out = np.zeros((num_expanded, rows.shape[1]), dtype=np.uint8)
    for t, positions in enumerate(token_topk_to_pos.tolist()):
        for pos in positions:
            if pos >= 0:
                out[pos] = rows[t]
    return torch.from_numpy(out).view(x.dtype).view(num_expanded, x.shape[1])


def expand_to_fused_with_sf(x, num_per_channels: int, token_topk_to_pos: torch.Tensor, pos_to_expert: torch.Tensor,
                            use_tma_aligned_col_major_sf: bool = False):
    """Row expansion of data and scales (tile_kernels/torch/expand_to_fused.py:42-91); the scales of the result
    are row-major, or a transposed view of a zero-initialised (hidden_sf, align(positions, 4)) buffer."""
    data, sf = x
    out = expand_to_fused(data, token_topk_to_pos, pos_to_expert)
    out_sf_rows = expand_to_fused(sf, token_topk_to_pos, pos_to_expert)
    if not use_tma_aligned_col_major_sf:
        return out, out_sf_rows
    num_expanded = pos_to_expert.shape[0]
    storage = torch.zeros((sf.shape[1], _ceil_div(num_expanded, 4) * 4), dtype=sf.dtype)
    storage[:, :num_expanded] = out_sf_rows.T
    return out, storage[:, :num_expanded].T


def expf(x: torch.Tensor) -> torch.Tensor:
    x = x.contiguous().float()
    y = torch.empty_like(x)
    lib().tkqo_expf_array(_vp(x.data_ptr()), _vp(y.data_ptr()), _i64(x.numel()))
    return y


def convert_array(x: torch.Tensor, fmt: str) -> torch.Tensor:
    """Element converters for the unit tests: fp32 -> codes ('e4m3' clamps to +-448 first)."""
    x = x.contiguous().float()
    if fmt == 'e5m6':
        y = torch.empty(x.shape, dtype=torch.int32)
        lib().tkqo_f32_to_e5m6_array(_vp(x.data_ptr()), _vp(y.data_ptr()), _i64(x.numel()))
        return y
    y = torch.empty(x.shape, dtype=torch.uint8)
    fn = lib().tkqo_f32_to_e4m3_array if fmt == 'e4m3' else lib().tkqo_f32_to_e2m1_array
    fn(_vp(x.data_ptr()), _vp(y.data_ptr()), _i64(x.numel()))
    return y
