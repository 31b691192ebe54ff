"""per_block_cast and per_channel_cast on the GPU against the oracle (parametrised as the reference's
tests/quant/test_per_block_cast.py:38-97 and test_per_channel_cast.py:22-55)."""
import pytest
import torch

from helpers import flags_id, to_host
from tilekernels_b200.testing import assert_equal, check_bias

pytestmark = pytest.mark.gpu

FLAGS = [(False, True, False), (True, True, True), (False, False, False)]


def _x(num_tokens, hidden, dtype):
    g = torch.Generator().manual_seed(num_tokens * 7 + hidden)
    x = torch.randn((num_tokens, hidden), generator=g)
    if num_tokens >= 256:
        x[128:256, :64] *= 50
        x[200] = 0
    return x.to(dtype)


@pytest.mark.parametrize('flags', FLAGS, ids=flags_id)
@pytest.mark.parametrize('block', [(128, 128), (32, 32), (128, 32), (32, 128)], ids=lambda b: f'{b[0]}x{b[1]}')
@pytest.mark.parametrize('fmt', ['e4m3', 'e2m1'])
@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float32], ids=['bf16', 'fp32'])
@pytest.mark.parametrize('num_tokens,hidden', [(4001, 576), (4001, 2048), (1025, 7168), (129, 2560), (31, 3072), (1, 64)])
def test_per_block_cast(oracle, cuda_device, num_tokens, hidden, dtype, fmt, block, flags):
    from tilekernels_b200 import quant
    col, rnd, ue = flags
    if block[0] != block[1] and (dtype == torch.float32 or ue):
        pytest.skip('mixed block shapes: covered for bf16 with fp32 scales')
    x_cpu = _x(num_tokens, hidden, dtype)
    x = x_cpu.to(cuda_device)
    kw = dict(use_tma_aligned_col_major_sf=col, round_sf=rnd, use_packed_ue8m0=ue)
    out, sf = quant.per_block_cast(x, fmt, block, **kw)
    out_ref, sf_ref = oracle.cast(x_cpu, fmt, block, **kw)
    assert_equal(to_host(sf), sf_ref)
    assert_equal(to_host(out), out_ref)
    if rnd and not col and num_tokens > 1000:
        check_bias(oracle.cast_back((out_ref, sf_ref), 'fp32', block), x_cpu.float())
    if not col:
        pre = quant.per_block_cast_with_precomputed_sf(x, fmt, block, sf=sf, **kw)
        assert_equal(to_host(pre), oracle.cast(x_cpu, fmt, block, sf=sf_ref))
    only = quant.per_block_cast_with_sf_only(x, fmt, block, **kw)
    assert_equal(to_host(only), sf_ref)


@pytest.mark.parametrize('round_sf', [False, True])
@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float32], ids=['bf16', 'fp32'])
@pytest.mark.parametrize('num_tokens,hidden', [(4096, 576), (4096, 2048), (1024, 7168), (128, 2560), (8064, 64), (256, 6144)])
def test_per_channel_cast(oracle, cuda_device, num_tokens, hidden, dtype, round_sf):
    from tilekernels_b200 import quant
    x_cpu = _x(num_tokens, hidden, dtype)
    out, sf = quant.per_channel_cast(x_cpu.to(cuda_device), 'e4m3', 128, round_sf)
    out_ref, sf_ref = oracle.cast(x_cpu, 'e4m3', (128, 1), round_sf=round_sf)
    assert_equal(to_host(out), out_ref)
    assert_equal(to_host(sf), sf_ref)
    if round_sf:
        check_bias(oracle.cast_back((out_ref, sf_ref), 'fp32', (128, 1)), x_cpu.float())


def test_tile_kernels_report_no_wait_failure(cuda_device):
    # the bounded tile wait never ran out during the tests above
    from tilekernels_b200 import _lib
    assert _lib.lib().tkq_device_error() == 0


def test_per_channel_cast_rejects_ragged_tokens(cuda_device):
    from tilekernels_b200 import quant
    with pytest.raises(AssertionError):
        quant.per_channel_cast(torch.zeros((100, 128), dtype=torch.bfloat16, device=cuda_device), 'e4m3', 128)


def _clamp_abs_ratio(x, max_ratio=2.0 ** 10):
    """Limit the dynamic range inside every 128 x 128 block so that the re-blocking is lossless."""
    a = x.abs().clamp_min(1e-30)
    T, H = x.shape
    pad = torch.nn.functional.pad(a, (0, (-H) % 128, 0, (-T) % 128), value=0)
    bmax = pad.view(pad.shape[0] // 128, 128, pad.shape[1] // 128, 128).amax(dim=(1, 3))
    floor = (bmax / max_ratio).repeat_interleave(128, 0)[:T].repeat_interleave(128, 1)[:, :H]
    return torch.where(a < floor, torch.sign(x) * floor + (x == 0) * floor, x)


@pytest.mark.parametrize('out_flags', [(False, True, False), (True, True, True)], ids=flags_id)
@pytest.mark.parametrize('in_flags', [(False, True, False), (True, True, True)], ids=flags_id)
@pytest.mark.parametrize('out_block', [(1, 128), (32, 32), (128, 128)], ids=lambda b: f'{b[0]}x{b[1]}')
@pytest.mark.parametrize('num_tokens,hidden', [(4001, 576), (4001, 7168), (129, 2048)])
def test_per_block_cast_lossless(oracle, cuda_device, num_tokens, hidden, out_block, in_flags, out_flags):
    """As the reference's tests/quant/test_per_block_cast_lossless.py:82-97: FP4 with (1, 32) power-of-two scales is
    re-blocked to FP8; both sides must dequantise to identical fp32 values.  Also bit-exact against the oracle."""
    from tilekernels_b200 import quant
    g = torch.Generator().manual_seed(num_tokens + hidden)
    x = _clamp_abs_ratio(torch.randn((num_tokens, hidden), generator=g) * 2.0 ** torch.randint(-20, 20, (1,), generator=g).item())
    icol, irnd, iue = in_flags
    ocol, ornd, oue = out_flags
    q_ref, qsf_ref = oracle.cast(x, 'e2m1', (1, 32), round_sf=irnd, use_tma_aligned_col_major_sf=icol, use_packed_ue8m0=iue)
    q, qsf = quant.per_token_cast(x.to(cuda_device), 'e2m1', 32, None, icol, irnd, iue)
    out, sf = quant.per_block_cast_lossless((q, qsf), 'e4m3', (1, 32), out_block, ocol, ornd, oue)
    out_ref, sf_ref = oracle.per_block_cast_lossless((q_ref, qsf_ref), (1, 32), out_block, ocol, oue)
    assert_equal(to_host(sf), sf_ref)
    assert_equal(to_host(out), out_ref)
    back_in = oracle.cast_back((q_ref, qsf_ref), 'fp32', (1, 32))
    back_out = oracle.cast_back((to_host(out), to_host(sf)), 'fp32', out_block)
    assert_equal(back_out, back_in)


def _lossless_block_pairs():
    yield (1, 16), (1, 32)
    yield (1, 16), (32, 32)
    yield (1, 16), (128, 128)
    yield (1, 32), (32, 128)
    yield (1, 32), (128, 32)
    yield (32, 32), (32, 32)
    yield (32, 32), (128, 128)
    yield (128, 128), (128, 128)


@pytest.mark.gpu
@pytest.mark.parametrize('flags', [(False, True, False), (True, True, True)], ids=flags_id)
@pytest.mark.parametrize('in_block,out_block', list(_lossless_block_pairs()), ids=lambda b: f'{b[0]}x{b[1]}')
@pytest.mark.parametrize('num_tokens,hidden', [(4001, 576), (129, 2048), (300, 7168)])
def test_per_block_cast_lossless_block_shapes(oracle, cuda_device, num_tokens, hidden, in_block, out_block, flags):
    """Input blocks other than (1, 32) -- 16 wide (two input scales inside a 32-value piece), 32 x 32, 128 x 128 -- and the
    mixed output blocks, in both scale layouts; bit-exact against the oracle and lossless."""
    from tilekernels_b200 import quant
    g = torch.Generator().manual_seed(num_tokens * 7 + hidden + in_block[1])
    x = _clamp_abs_ratio(torch.randn((num_tokens, hidden), generator=g) * 2.0 ** torch.randint(-20, 20, (1,), generator=g).item())
    col, rnd, ue = flags
    q_ref, qsf_ref = oracle.cast(x, 'e2m1', in_block, round_sf=rnd, use_tma_aligned_col_major_sf=col, use_packed_ue8m0=ue)
    if in_block[0] == 1:
        q, qsf = quant.per_token_cast(x.to(cuda_device), 'e2m1', in_block[1], None, col, rnd, ue)
    else:
        q, qsf = quant.per_block_cast(x.to(cuda_device), 'e2m1', in_block, col, rnd, ue)
    assert_equal(to_host(q), q_ref)
    assert_equal(to_host(qsf), qsf_ref)
    out, sf = quant.per_block_cast_lossless((q, qsf), 'e4m3', in_block, out_block, col, rnd, ue)
    out_ref, sf_ref = oracle.per_block_cast_lossless((q_ref, qsf_ref), in_block, out_block, col, ue)
    assert_equal(to_host(sf), sf_ref)
    assert_equal(to_host(out), out_ref)
    back_in = oracle.cast_back((q_ref, qsf_ref), 'fp32', in_block)
    back_out = oracle.cast_back((to_host(out), to_host(sf)), 'fp32', out_block)
    assert_equal(back_out, back_in)



def test_per_block_cast_lossless_reports_range_violation(cuda_device):
    """Where the reference's kernel asserts on the device (an input scale more than 2^5 below its output block's
    scale, tile_kernels/quant/per_block_cast_lossless_kernel.py:128), this library finishes the cast and raises
    TKQ_DEVICE_LOSSLESS_RANGE (2), once, through tkq_device_error()."""
    from tilekernels_b200 import _lib, quant
    lib = _lib.lib()
    assert lib.tkq_device_error() == 0
    g = torch.Generator().manual_seed(5)
    x = torch.randn((256, 256), generator=g)
    q, qsf = quant.per_token_cast(x.to(cuda_device), 'e2m1', 32, None, False, True, False)
    quant.per_block_cast_lossless((q, qsf), 'e4m3', (1, 32), (128, 128), False, True, False)
    assert lib.tkq_device_error() == 0              # ordinary data: every block within range
    x[:, 32:64] *= 2.0 ** -12                        # one 32-wide input block 2^12 below its neighbours
    q, qsf = quant.per_token_cast(x.to(cuda_device), 'e2m1', 32, None, False, True, False)
    quant.per_block_cast_lossless((q, qsf), 'e4m3', (1, 32), (128, 128), False, True, False)
    assert lib.tkq_device_error() == 2
    assert lib.tkq_device_error() == 0


@pytest.mark.parametrize('op', ['per_block', 'per_channel', 'per_channel_gather'])
def test_direct_tile_kernels_with_16_byte_aligned_input(oracle, cuda_device, op):
    """The direct kernels read 32 bytes per lane with one 256-bit load when the tensor starts on a 32-byte boundary
    and with two 128-bit loads otherwise: a contiguous tensor that starts 16 bytes into an allocation takes the second
    form and must give the same bytes."""
    from tilekernels_b200 import quant
    g = torch.Generator().manual_seed(77)
    x_cpu = torch.randn((384, 576), generator=g).to(torch.bfloat16)
    buf = torch.empty(x_cpu.numel() + 8, dtype=torch.bfloat16, device=cuda_device)
    x = buf[8:].view(384, 576)
    x.copy_(x_cpu)
    assert x.data_ptr() % 32 == 16 and x.is_contiguous()
    if op == 'per_block':
        out, sf = quant.per_block_cast(x, 'e4m3', (128, 128))
        out_ref, sf_ref = oracle.cast(x_cpu, 'e4m3', (128, 128))
    elif op == 'per_channel':
        out, sf = quant.per_channel_cast(x, 'e4m3', 128)
        out_ref, sf_ref = oracle.cast(x_cpu, 'e4m3', (128, 1))
    else:
        pos = torch.randint(0, 384, (256,), generator=g, dtype=torch.int32)
        pos[::5] = -1
        out, sf = quant.per_channel_cast_fused(x, 'e4m3', 128, False, None, pos.to(cuda_device))
        gathered = torch.where((pos >= 0).unsqueeze(-1), x_cpu[pos.clamp_min(0).long()], torch.zeros((), dtype=torch.bfloat16))
        out_ref, sf_ref = oracle.cast(gathered, 'e4m3', (128, 1))
    assert_equal(to_host(sf), sf_ref)
    assert_equal(to_host(out), out_ref)
