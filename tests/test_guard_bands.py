"""Out-of-bounds stores, checked without a memory checker: every output of a cast is placed inside a larger device
buffer filled with 0xA5, the entry point is called through the raw C ABI with the interior pointer, and the WHOLE
buffer is compared with what it must hold afterwards: the oracle's bytes at the logical positions, 0xA5 everywhere
else -- in front of and behind the output, and in the padding of the column-major scale layouts (token padding up
to the 16-byte pitch is never written).  Ragged shapes: tokens 1, 3, 127, 129, 4001; hidden 64 and 576."""
import ctypes

import pytest
import torch

from helpers import flags_id

pytestmark = pytest.mark.gpu

GUARD = 4096          # bytes in front of and behind every output
FILL = 0xA5
TOKENS = [1, 3, 127, 129, 4001]
FLAG_SETS = [(False, False, False), (True, True, False), (True, True, True)]  # (col_major, round_sf, ue8m0)


def _ceil_div(a, b):
    return (a + b - 1) // b


def _align(a, b):
    return _ceil_div(a, b) * b


class Guarded:
    """`nbytes` of device memory surrounded by guard bytes, everything pre-filled with FILL."""

    def __init__(self, nbytes: int, device):
        self.nbytes = nbytes
        self.buf = torch.full((GUARD + nbytes + GUARD,), FILL, dtype=torch.uint8, device=device)

    @property
    def ptr(self) -> int:
        return self.buf.data_ptr() + GUARD

    def check(self, expected_interior: torch.Tensor, what: str) -> None:
        """expected_interior: uint8 CPU tensor of nbytes (FILL where nothing may be written)."""
        got = self.buf.cpu()
        want = torch.full_like(got, FILL)
        want[GUARD:GUARD + self.nbytes] = expected_interior
        if not torch.equal(got, want):
            bad = torch.nonzero(got != want).flatten()
            where = [int(b) - GUARD for b in bad[:6]]
            raise AssertionError(f'{what}: {bad.numel()} wrong bytes, first at offsets {where} relative to the output start '
                                 f'(logical size {self.nbytes})')


def _sf_geometry(nm: int, nk: int, col: bool, ue: bool):
    """(storage bytes, sf_stride argument) of the scale layouts of include/tkquant.h."""
    if ue:
        pitch = _align(4 * nm, 16)
        return _ceil_div(nk, 4) * pitch, pitch
    if col:
        pitch = _align(nm, 4)
        return nk * pitch * 4, pitch
    return nm * nk * 4, nk


def _expected_sf(sf_ref: torch.Tensor, nm: int, nk: int, col: bool, ue: bool) -> torch.Tensor:
    """The scale storage as bytes: the oracle's values at their places, FILL in the padding."""
    nbytes, stride = _sf_geometry(nm, nk, col, ue)
    store = torch.full((nbytes,), FILL, dtype=torch.uint8)
    if ue:
        words = store.view(torch.int32).view(_ceil_div(nk, 4), stride // 4)
        words[:, :nm] = sf_ref.T          # int32 [nm, ceil(nk / 4)], padding bytes of the last word are zero
    elif col:
        store.view(torch.float32).view(nk, stride)[:, :nm] = sf_ref.T
    else:
        store.view(torch.float32).view(nm, nk)[:] = sf_ref
    return store


def _flags(col, rnd, ue):
    return (1 if rnd else 0) | (2 if col else 0) | (4 if ue else 0)


def _raw(t: torch.Tensor) -> torch.Tensor:
    return t.contiguous().view(torch.uint8).flatten()


@pytest.mark.parametrize('flags', FLAG_SETS, ids=flags_id)
@pytest.mark.parametrize('fmt,group', [('e4m3', 32), ('e4m3', 0), ('e2m1', 32)])
@pytest.mark.parametrize('hidden', [64, 576])
@pytest.mark.parametrize('num_tokens', TOKENS)
def test_per_token_cast_guard_bands(oracle, cuda_device, num_tokens, hidden, fmt, group, flags):
    from tilekernels_b200 import _lib
    col, rnd, ue = flags
    group = group or hidden
    if group == hidden and col:
        pytest.skip('one scale per token is used with row-major scales')
    x = torch.randn((num_tokens, hidden), generator=torch.Generator().manual_seed(num_tokens + hidden)).to(torch.bfloat16)
    out_ref, sf_ref = oracle.cast(x, fmt, (1, group), round_sf=rnd, use_tma_aligned_col_major_sf=col, use_packed_ue8m0=ue)
    nk = _ceil_div(hidden, group)
    sf_bytes, sf_stride = _sf_geometry(num_tokens, nk, col, ue)
    out = Guarded(num_tokens * (hidden if fmt == 'e4m3' else hidden // 2), cuda_device)
    sf = Guarded(sf_bytes, cuda_device)
    xd = x.to(cuda_device)
    rc = _lib.lib().tkq_per_token_cast(xd.data_ptr(), 0, num_tokens, hidden, hidden, 0 if fmt == 'e4m3' else 1, group,
                                       _flags(col, rnd, ue), out.ptr, sf.ptr, sf_stride, None)
    assert rc == 0, _lib.lib().tkq_last_error_string()
    torch.cuda.synchronize()
    out.check(_raw(out_ref), 'per_token_cast data')
    sf.check(_expected_sf(sf_ref, num_tokens, nk, col, ue), 'per_token_cast scales')


@pytest.mark.parametrize('flags', FLAG_SETS, ids=flags_id)
@pytest.mark.parametrize('hidden', [64, 576])
@pytest.mark.parametrize('num_tokens', TOKENS)
def test_e5m6_guard_bands(oracle, cuda_device, num_tokens, hidden, flags):
    from tilekernels_b200 import _lib
    col, rnd, ue = flags
    x = torch.randn((num_tokens, hidden), generator=torch.Generator().manual_seed(7 + num_tokens)).to(torch.bfloat16)
    out_ref, sf_ref = oracle.cast_to_e5m6(x, hidden, col, rnd, ue)
    sf_bytes, sf_stride = _sf_geometry(num_tokens, 1, col, ue)
    out = Guarded(num_tokens * hidden // 8 * 12, cuda_device)
    sf = Guarded(sf_bytes, cuda_device)
    xd = x.to(cuda_device)
    rc = _lib.lib().tkq_per_token_cast_e5m6(xd.data_ptr(), 0, num_tokens, hidden, hidden, _flags(col, rnd, ue), out.ptr, sf.ptr,
                                            sf_stride, None)
    assert rc == 0, _lib.lib().tkq_last_error_string()
    torch.cuda.synchronize()
    out.check(_raw(out_ref), 'e5m6 data')
    sf.check(_expected_sf(sf_ref, num_tokens, 1, col, ue), 'e5m6 scales')


@pytest.mark.parametrize('flags', FLAG_SETS, ids=flags_id)
@pytest.mark.parametrize('block', [128, 32])
@pytest.mark.parametrize('hidden', [64, 576])
@pytest.mark.parametrize('num_tokens', TOKENS)
def test_per_block_cast_guard_bands(oracle, cuda_device, num_tokens, hidden, block, flags):
    from tilekernels_b200 import _lib
    col, rnd, ue = flags
    x = torch.randn((num_tokens, hidden), generator=torch.Generator().manual_seed(11 + num_tokens)).to(torch.bfloat16)
    out_ref, sf_ref = oracle.cast(x, 'e4m3', (block, block), round_sf=rnd, use_tma_aligned_col_major_sf=col, use_packed_ue8m0=ue)
    nm, nk = _ceil_div(num_tokens, block), _ceil_div(hidden, block)
    sf_bytes, sf_stride = _sf_geometry(nm, nk, col, ue)
    out = Guarded(num_tokens * hidden, cuda_device)
    sf = Guarded(sf_bytes, cuda_device)
    xd = x.to(cuda_device)
    rc = _lib.lib().tkq_per_block_cast(xd.data_ptr(), 0, num_tokens, hidden, 0, block, block, _flags(col, rnd, ue), out.ptr, sf.ptr,
                                       sf_stride, None)
    assert rc == 0, _lib.lib().tkq_last_error_string()
    torch.cuda.synchronize()
    out.check(_raw(out_ref), 'per_block_cast data')
    sf.check(_expected_sf(sf_ref, nm, nk, col, ue), 'per_block_cast scales')


@pytest.mark.parametrize('hidden', [64, 576])
@pytest.mark.parametrize('num_tokens', [128, 384])
def test_per_channel_cast_guard_bands(oracle, cuda_device, num_tokens, hidden):
    from tilekernels_b200 import _lib
    x = torch.randn((num_tokens, hidden), generator=torch.Generator().manual_seed(13)).to(torch.bfloat16)
    out_ref, sf_ref = oracle.cast(x, 'e4m3', (128, 1))
    out = Guarded(num_tokens * hidden, cuda_device)
    sf = Guarded(num_tokens // 128 * hidden * 4, cuda_device)
    xd = x.to(cuda_device)
    rc = _lib.lib().tkq_per_channel_cast(xd.data_ptr(), 0, num_tokens, hidden, 0, out.ptr, sf.ptr, None)
    assert rc == 0, _lib.lib().tkq_last_error_string()
    torch.cuda.synchronize()
    out.check(_raw(out_ref), 'per_channel_cast data')
    sf.check(_raw(sf_ref), 'per_channel_cast scales')


@pytest.mark.parametrize('flags', FLAG_SETS, ids=flags_id)
@pytest.mark.parametrize('hidden', [128, 1152])
@pytest.mark.parametrize('num_tokens', TOKENS)
def test_swiglu_cast_guard_bands(oracle, cuda_device, num_tokens, hidden, flags):
    """hidden 128 takes the register kernel, 1152 the staged kernel with a partly filled row segment.  Scales must be
    exact; a data byte may differ from the oracle by one code step (approximate kernel), never in a guard byte."""
    from tilekernels_b200 import _lib
    col, rnd, ue = flags
    x = torch.randn((num_tokens, 2 * hidden), generator=torch.Generator().manual_seed(17 + num_tokens)).to(torch.bfloat16)
    out_ref, sf_ref = oracle.cast(oracle.swiglu_forward(x), 'e4m3', (1, 128), round_sf=rnd, use_tma_aligned_col_major_sf=col,
                                  use_packed_ue8m0=ue)
    nk = hidden // 128
    sf_bytes, sf_stride = _sf_geometry(num_tokens, nk, col, ue)
    out = Guarded(num_tokens * hidden, cuda_device)
    sf = Guarded(sf_bytes, cuda_device)
    xd = x.to(cuda_device)
    rc = _lib.lib().tkq_swiglu_forward_and_per_token_cast(xd.data_ptr(), 0, num_tokens, hidden, 128, None, None, None,
                                                          ctypes.c_float(-1.0), None, ctypes.c_float(-1.0), 0,
                                                          _flags(col, rnd, ue), out.ptr, sf.ptr, sf_stride, None)
    assert rc == 0, _lib.lib().tkq_last_error_string()
    torch.cuda.synchronize()
    sf.check(_expected_sf(sf_ref, num_tokens, nk, col, ue), 'swiglu cast scales')
    got = out.buf.cpu()
    interior = got[GUARD:GUARD + out.nbytes]
    step = (interior.to(torch.int32) - _raw(out_ref).to(torch.int32)).abs()
    assert int(step.max()) <= 1 and int((step > 0).sum()) <= max(1, int(1e-4 * step.numel()))
    out.check(interior, 'swiglu cast data (guard bytes)')


@pytest.mark.parametrize('out_dtype', [torch.bfloat16, torch.float32])
@pytest.mark.parametrize('hidden', [64, 576])
@pytest.mark.parametrize('num_tokens', TOKENS)
def test_cast_back_guard_bands(oracle, cuda_device, num_tokens, hidden, out_dtype):
    from tilekernels_b200 import _lib
    x = torch.randn((num_tokens, hidden), generator=torch.Generator().manual_seed(19 + num_tokens)).to(torch.bfloat16)
    q, qsf = oracle.cast(x, 'e4m3', (1, 32), round_sf=True)
    want = oracle.cast_back((q, qsf), 'fp32', (1, 32)).to(out_dtype)
    out = Guarded(num_tokens * hidden * (2 if out_dtype == torch.bfloat16 else 4), cuda_device)
    qd, sd = q.to(cuda_device), qsf.to(cuda_device)
    rc = _lib.lib().tkq_cast_back(qd.data_ptr(), 0, sd.data_ptr(), 0, hidden // 32, 1, 32, num_tokens, hidden,
                                  0 if out_dtype == torch.bfloat16 else 1, out.ptr, None)
    assert rc == 0, _lib.lib().tkq_last_error_string()
    torch.cuda.synchronize()
    out.check(_raw(want), 'cast_back data')


def _device_sf(sf_ref: torch.Tensor, nm: int, nk: int, col: bool, ue: bool, device):
    """An input scale tensor in device storage laid out as the C ABI reads it; returns (tensor, sf_stride argument)."""
    store = _expected_sf(sf_ref, nm, nk, col, ue)
    return store.to(device), _sf_geometry(nm, nk, col, ue)[1]


@pytest.mark.parametrize('flags', [(False, True, False), (True, True, True)], ids=flags_id)
@pytest.mark.parametrize('in_fmt,in_block', [('e4m3', (128, 128)), ('e4m3', (1, 128)), ('e2m1', (1, 32))], ids=lambda v: str(v).replace(' ', ''))
@pytest.mark.parametrize('hidden', [576, 1024, 2048])
@pytest.mark.parametrize('num_tokens', [1, 127, 129, 1031])
def test_requantising_cast_guard_bands(oracle, cuda_device, num_tokens, hidden, in_fmt, in_block, flags):
    """tkq_per_token_cast_quantized to e4m3 with groups of 128: rows of whole 1024-value steps take the kernel with 32 values
    per lane, the others the general one; the same scale layout on both sides."""
    from tilekernels_b200 import _lib
    col, rnd, ue = flags
    x = torch.randn((num_tokens, hidden), generator=torch.Generator().manual_seed(31 + num_tokens + hidden)).to(torch.bfloat16)
    kw = dict(round_sf=rnd, use_tma_aligned_col_major_sf=col, use_packed_ue8m0=ue)
    q, qsf = oracle.cast(x, in_fmt, in_block, **kw)
    out_ref, sf_ref = oracle.cast((q, qsf), 'e4m3', (1, 128), x_block_size=in_block, **kw)
    nm_in, nk_in = _ceil_div(num_tokens, in_block[0]), _ceil_div(hidden, in_block[1])
    in_sf, in_stride = _device_sf(qsf, nm_in, nk_in, col, ue, cuda_device)
    nk = _ceil_div(hidden, 128)
    sf_bytes, sf_stride = _sf_geometry(num_tokens, nk, col, ue)
    out, sf = Guarded(num_tokens * hidden, cuda_device), Guarded(sf_bytes, cuda_device)
    qd = q.to(cuda_device)
    sf_flags = _flags(col, False, ue)
    rc = _lib.lib().tkq_per_token_cast_quantized(qd.data_ptr(), 0 if in_fmt == 'e4m3' else 1, in_sf.data_ptr(), sf_flags, in_stride, in_block[0],
                                                 in_block[1], num_tokens, hidden, hidden, 0, 128, _flags(col, rnd, ue), out.ptr, sf.ptr,
                                                 sf_stride, None)
    assert rc == 0, _lib.lib().tkq_last_error_string()
    torch.cuda.synchronize()
    out.check(_raw(out_ref), 'requantising cast data')
    sf.check(_expected_sf(sf_ref, num_tokens, nk, col, ue), 'requantising cast scales')


@pytest.mark.parametrize('flags', [(False, True, False), (True, True, False), (True, True, True)], ids=flags_id)
@pytest.mark.parametrize('out_block', [(128, 128), (32, 32), (1, 128)], ids=lambda b: f'{b[0]}x{b[1]}')
@pytest.mark.parametrize('hidden', [64, 576, 1280])
@pytest.mark.parametrize('num_tokens', TOKENS)
def test_lossless_cast_guard_bands(oracle, cuda_device, num_tokens, hidden, out_block, flags):
    """tkq_per_block_cast_lossless on ragged shapes (partial 128 x 256 tiles in both directions)."""
    from tilekernels_b200 import _lib
    col, _, ue = flags
    x = torch.randn((num_tokens, hidden), generator=torch.Generator().manual_seed(37 + num_tokens + hidden)).to(torch.bfloat16)
    q, qsf = oracle.cast(x, 'e2m1', (1, 32), round_sf=True)
    out_ref, sf_ref = oracle.per_block_cast_lossless((q, qsf), (1, 32), out_block, col, ue)
    nm, nk = _ceil_div(num_tokens, out_block[0]), _ceil_div(hidden, out_block[1])
    sf_bytes, sf_stride = _sf_geometry(nm, nk, col, ue)
    out, sf = Guarded(num_tokens * hidden, cuda_device), Guarded(sf_bytes, cuda_device)
    qd, sd = q.to(cuda_device), qsf.contiguous().to(cuda_device)
    rc = _lib.lib().tkq_per_block_cast_lossless(qd.data_ptr(), sd.data_ptr(), 0, hidden // 32, 1, 32, num_tokens, hidden, hidden, out_block[0],
                                                out_block[1], _flags(col, False, ue), out.ptr, sf.ptr, sf_stride, None)
    assert rc == 0, _lib.lib().tkq_last_error_string()
    torch.cuda.synchronize()
    out.check(_raw(out_ref), 'lossless cast data')
    sf.check(_expected_sf(sf_ref, nm, nk, col, ue), 'lossless cast scales')


@pytest.mark.parametrize('col', [False, True], ids=['row-major', 'col-major'])
@pytest.mark.parametrize('row_bytes', [48, 576, 2064])
@pytest.mark.parametrize('num_tokens,num_topk,num_pad', [(1, 1, 3), (33, 2, 7), (257, 6, 41)])
def test_expand_guard_bands(oracle, cuda_device, num_tokens, num_topk, num_pad, row_bytes, col):
    """tkq_expand_to_fused with scale words: rows of a whole number of 16-byte pieces (not of 32), padded positions
    cleared, nothing written behind the last expanded row or in the padding of the column-major scale buffer."""
    from tilekernels_b200 import _lib
    gen = torch.Generator().manual_seed(41 + num_tokens + row_bytes)
    entries = num_tokens * num_topk
    routed = torch.rand(entries, generator=gen) > 0.2
    num_routed = int(routed.sum().item())
    num_expanded = num_routed + num_pad
    positions = torch.randperm(num_expanded, generator=gen)[:num_routed].to(torch.int32)
    t2p = torch.full((entries,), -1, dtype=torch.int32)
    t2p[routed] = positions
    p2e = torch.full((num_expanded,), -1, dtype=torch.int32)
    p2e[positions.long()] = 0
    t2p = t2p.view(num_tokens, num_topk)
    sf_words = 5
    x = torch.randint(0, 256, (num_tokens, row_bytes), generator=gen, dtype=torch.int32).to(torch.uint8)
    x_sf = torch.randint(1, 2 ** 31 - 1, (num_tokens, sf_words), generator=gen, dtype=torch.int64).to(torch.int32)
    out_ref = oracle.expand_to_fused(x, t2p, p2e)
    sf_rows = oracle.expand_to_fused(x_sf, t2p, p2e)            # [num_expanded, sf_words]
    out = Guarded(num_expanded * row_bytes, cuda_device)
    stride = _align(num_expanded, 4) if col else sf_words
    sf = Guarded((sf_words * stride if col else num_expanded * sf_words) * 4, cuda_device)
    want_sf = torch.full((sf.nbytes,), FILL, dtype=torch.uint8)
    if col:
        want_sf.view(torch.int32).view(sf_words, stride)[:, :num_expanded] = sf_rows.T
    else:
        want_sf.view(torch.int32).view(num_expanded, sf_words)[:] = sf_rows
    xd, sd, td, pd = x.to(cuda_device), x_sf.to(cuda_device), t2p.to(cuda_device), p2e.to(cuda_device)
    rc = _lib.lib().tkq_expand_to_fused(xd.data_ptr(), num_tokens, row_bytes, sd.data_ptr(), sf_words, td.data_ptr(), num_topk, pd.data_ptr(),
                                        num_expanded, 2 if col else 0, out.ptr, sf.ptr, stride, None)
    assert rc == 0, _lib.lib().tkq_last_error_string()
    torch.cuda.synchronize()
    out.check(_raw(out_ref), 'expand data')
    sf.check(want_sf, 'expand scales')


@pytest.mark.parametrize('num_per_tokens', [32, 128])
@pytest.mark.parametrize('hidden', [64, 576])
@pytest.mark.parametrize('num_tokens', [128, 384])
def test_transposing_cast_guard_bands(oracle, cuda_device, num_tokens, hidden, num_per_tokens):
    """tkq_per_channel_cast_and_transpose: the transposed data and the [tokens / n, hidden] scales."""
    from tilekernels_b200 import _lib
    x = torch.randn((num_tokens, hidden), generator=torch.Generator().manual_seed(43 + num_tokens + hidden)).to(torch.bfloat16)
    out_ref, sf_ref = oracle.cast(x, 'e4m3', (num_per_tokens, 1))
    out = Guarded(num_tokens * hidden, cuda_device)
    sf = Guarded(num_tokens // num_per_tokens * hidden * 4, cuda_device)
    xd = x.to(cuda_device)
    rc = _lib.lib().tkq_per_channel_cast_and_transpose(xd.data_ptr(), num_tokens, hidden, num_per_tokens, 0, out.ptr, sf.ptr, None)
    assert rc == 0, _lib.lib().tkq_last_error_string()
    torch.cuda.synchronize()
    out.check(_raw(out_ref.T.contiguous()), 'transposing cast data')
    sf.check(_raw(sf_ref), 'transposing cast scales')


@pytest.mark.parametrize('hidden', [64, 576])
@pytest.mark.parametrize('num_out', [16, 144, 400])
def test_gathering_channel_cast_guard_bands(oracle, cuda_device, num_out, hidden):
    """tkq_per_channel_cast_fused with pos_to_token: output rows in multiples of 16 (a partial last band of 128), negative
    entries give rows of zeros."""
    from tilekernels_b200 import _lib
    gen = torch.Generator().manual_seed(47 + num_out + hidden)
    num_in = 200
    x = torch.randn((num_in, hidden), generator=gen).to(torch.bfloat16)
    pos = torch.randint(0, num_in, (num_out,), generator=gen, dtype=torch.int32)
    pos[::7] = -1
    out_ref, sf_ref = oracle.per_channel_cast_fused(x, 128, None, False, pos)
    nm = _ceil_div(num_out, 128)
    out, sf = Guarded(num_out * hidden, cuda_device), Guarded(nm * hidden * 4, cuda_device)
    xd, pd = x.to(cuda_device), pos.to(cuda_device)
    rc = _lib.lib().tkq_per_channel_cast_fused(xd.data_ptr(), 0, None, pd.data_ptr(), num_in, num_out, hidden, 0, out.ptr, sf.ptr, None)
    assert rc == 0, _lib.lib().tkq_last_error_string()
    torch.cuda.synchronize()
    out.check(_raw(out_ref), 'gathering per-channel cast data')
    sf.check(_raw(sf_ref), 'gathering per-channel cast scales')


@pytest.mark.parametrize('group', [32, 128])
@pytest.mark.parametrize('hidden', [128, 384])
@pytest.mark.parametrize('num_tokens,num_topk,num_pad', [(1, 1, 0), (37, 2, 5), (130, 3, 9)])
def test_swiglu_backward_guard_bands(oracle, cuda_device, num_tokens, num_topk, num_pad, hidden, group):
    """tkq_swiglu_backward_and_per_token_cast: its four row-shaped outputs (bf16 activation, FP8 gradient with scales,
    bf16 gradient) inside guard bands; weight_grad (a sum in another order) is compared in the kernel's own test."""
    from tilekernels_b200 import _lib
    gen = torch.Generator().manual_seed(53 + num_tokens + hidden + group)
    entries = num_tokens * num_topk
    routed = torch.rand(entries, generator=gen) > 0.2
    num_routed = int(routed.sum().item())
    rows = num_routed + num_pad
    if rows == 0:
        pytest.skip('nothing routed')
    positions = torch.randperm(rows, generator=gen)[:num_routed].to(torch.int32)
    t2p = torch.full((entries,), -1, dtype=torch.int32)
    t2p[routed] = positions
    pos = torch.full((rows,), -1, dtype=torch.int32)
    pos[positions.long()] = torch.nonzero(routed).flatten().to(torch.int32)
    t2p = t2p.view(num_tokens, num_topk)
    xb = (torch.randn((rows, 2 * hidden), generator=gen) * 2).to(torch.bfloat16)
    q, qsf = oracle.cast(xb, 'e4m3', (1, group))
    d = torch.randn((rows, hidden), generator=gen).to(torch.bfloat16)
    w = torch.rand((num_tokens, num_topk), generator=gen)
    out_ref, x_grad_ref, _ = oracle.swiglu_backward((q, qsf), d, w, pos, t2p, group, None)
    fp8_ref, sf_ref = oracle.cast(x_grad_ref, 'e4m3', (1, group), round_sf=True)
    out = Guarded(rows * hidden * 2, cuda_device)
    fp8 = Guarded(rows * 2 * hidden, cuda_device)
    sf = Guarded(rows * (2 * hidden // group) * 4, cuda_device)
    x_grad = Guarded(rows * 2 * hidden * 2, cuda_device)
    w_grad = torch.zeros((num_tokens, num_topk), dtype=torch.float32, device=cuda_device)
    qd, sd, dd, wd, pd, td = (t.contiguous().to(cuda_device) for t in (q, qsf, d, w, pos, t2p))
    rc = _lib.lib().tkq_swiglu_backward_and_per_token_cast(qd.data_ptr(), sd.data_ptr(), dd.data_ptr(), wd.data_ptr(), pd.data_ptr(), td.data_ptr(),
                                                           rows, hidden, num_tokens, num_topk, group, -1.0, 1, out.ptr, fp8.ptr, sf.ptr, x_grad.ptr,
                                                           w_grad.data_ptr(), None)
    assert rc == 0, _lib.lib().tkq_last_error_string()
    torch.cuda.synchronize()
    out.check(_raw(out_ref.bfloat16()), 'backward activation')
    x_grad.check(_raw(x_grad_ref.bfloat16()), 'backward gradient (bf16)')
    fp8.check(_raw(fp8_ref), 'backward gradient (FP8)')
    sf.check(_raw(sf_ref), 'backward gradient scales')


@pytest.mark.parametrize('transpose', [0, 1])
@pytest.mark.parametrize('num_per_tokens', [32, 128])
@pytest.mark.parametrize('hidden', [64, 320])
@pytest.mark.parametrize('num_tokens', [128, 384])
def test_swiglu_channel_cast_guard_bands(oracle, cuda_device, num_tokens, hidden, num_per_tokens, transpose):
    """tkq_swiglu_forward_and_per_channel_cast: the bf16-rounded activation cast per (n tokens x 1 channel), plain or
    transposed."""
    from tilekernels_b200 import _lib
    x = torch.randn((num_tokens, 2 * hidden), generator=torch.Generator().manual_seed(59 + num_tokens + hidden)).to(torch.bfloat16)
    act = oracle.swiglu_forward(x).to(torch.bfloat16)
    out_ref, sf_ref = oracle.cast(act, 'e4m3', (num_per_tokens, 1))
    out = Guarded(num_tokens * hidden, cuda_device)
    sf = Guarded(num_tokens // num_per_tokens * hidden * 4, cuda_device)
    xd = x.to(cuda_device)
    rc = _lib.lib().tkq_swiglu_forward_and_per_channel_cast(xd.data_ptr(), num_tokens, hidden, num_per_tokens, transpose, -1.0, 0, out.ptr, sf.ptr, None)
    assert rc == 0, _lib.lib().tkq_last_error_string()
    torch.cuda.synchronize()
    out.check(_raw(out_ref.T.contiguous() if transpose else out_ref), 'SwiGLU per-channel cast data')
    sf.check(_raw(sf_ref), 'SwiGLU per-channel cast scales')
