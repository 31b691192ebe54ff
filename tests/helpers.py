"""Shared helpers of the test-suite: golden-fixture access and device-to-host comparison."""
import json
import os

import numpy as np
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), 'golden')
FLAG_SETS = [(False, False, False), (False, True, False), (True, True, True)]  # (col_major, round_sf, ue8m0)

_DTYPES = {'bfloat16': torch.bfloat16, 'float32': torch.float32, 'float8_e4m3fn': torch.float8_e4m3fn, 'int8': torch.int8,
           'uint8': torch.uint8, 'int32': torch.int32, 'int64': torch.int64}
_cache = {}


def golden(name: str):
    if name not in _cache:
        _cache[name] = np.load(os.path.join(GOLDEN, name + '.npz'))
    return _cache[name]


def golden_tensor(store, key: str) -> torch.Tensor:
    """Rebuild a stored tensor with its dtype, shape and strides."""
    m = json.loads(str(store[key + '.meta']))
    dtype, shape, stride = _DTYPES[m['dtype']], m['shape'], m['stride']
    dense = torch.from_numpy(store[key + '.bytes'].copy()).view(dtype).reshape(shape)
    if list(dense.stride()) == stride or dense.numel() == 0:
        return dense
    # strided storage (column-major scales): lay the values out with the stored strides
    span = 1 + sum((n - 1) * s for n, s in zip(shape, stride))
    out = torch.zeros(span, dtype=dtype).as_strided(shape, stride)
    out.copy_(dense)
    return out


def to_host(t: torch.Tensor) -> torch.Tensor:
    """Device tensor -> CPU tensor with the same strides (Tensor.cpu() would compact padded layouts)."""
    if t.device.type == 'cpu':
        return t
    if t.numel() == 0:
        return torch.empty_strided(t.shape, t.stride(), dtype=t.dtype)
    span = 1 + sum((n - 1) * s for n, s in zip(t.shape, t.stride()))
    out = torch.zeros(span, dtype=t.dtype).as_strided(t.shape, t.stride())
    out.copy_(t)
    return out


def flags_id(flags) -> str:
    return ''.join(str(int(f)) for f in flags)


def swiglu_cast_differences(out: torch.Tensor, sf: torch.Tensor, out_ref: torch.Tensor, sf_ref: torch.Tensor, group: int,
                            sf_to_float) -> dict:
    """Counts behind the acceptance rule of the fused SwiGLU cast: scales identical, FP8 codes at most one code
    apart on at most 1e-4 of the elements, dequantised values of equal codes within 1e-3 (relative).

    All four tensors on the CPU, scales in the same layout; `sf_to_float` turns either scale format into fp32."""
    assert out.shape == out_ref.shape and sf.shape == sf_ref.shape and sf.dtype == sf_ref.dtype
    s, s_ref = sf_to_float(sf), sf_to_float(sf_ref)
    ulp = (s.contiguous().view(torch.int32) - s_ref.contiguous().view(torch.int32)).abs()
    a, b = out.contiguous().view(torch.uint8).to(torch.int32), out_ref.contiguous().view(torch.uint8).to(torch.int32)
    diff = (a - b).abs()
    hidden = out.shape[1]
    dq = out.float() * s.repeat_interleave(group, dim=1)[:, :hidden]
    dq_ref = out_ref.float() * s_ref.repeat_interleave(group, dim=1)[:, :hidden]
    same = diff == 0
    rel = ((dq - dq_ref).abs() / dq_ref.abs().clamp_min(1e-30))[same]
    return {
        'scales': ulp.numel(), 'scales_differing': int((ulp > 0).sum()), 'scale_max_ulp': int(ulp.max()) if ulp.numel() else 0,
        'codes': diff.numel(), 'codes_differing': int((diff > 0).sum()), 'code_max_step': int(diff.max()) if diff.numel() else 0,
        'dequant_max_rel_equal_codes': float(rel.max()) if rel.numel() else 0.0,
    }
