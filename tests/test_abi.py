"""The C-ABI library without a GPU: it loads, exports every symbol the header declares, and rejects bad
arguments with the documented negative codes before touching the device."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope='module')
def lib():
    from tilekernels_b200 import _lib, build
    build.build()
    return _lib.lib()


def _declared_functions():
    text = open(os.path.join(ROOT, 'include', 'tkquant.h')).read()
    text = re.sub(r'/\*.*?\*/', '', text, flags=re.S)
    return sorted(set(re.findall(r'\b(tkq_[a-z0-9_]+)\s*\(', text)))


def test_header_symbols_are_exported(lib):
    names = _declared_functions()
    assert 'tkq_per_token_cast' in names and len(names) >= 8
    for name in names:
        assert hasattr(lib, name), f'{name} is declared in include/tkquant.h but not exported'


def test_binding_covers_header():
    from tilekernels_b200 import _lib
    assert set(_declared_functions()) == set(_lib.SIGNATURES) | {'tkq_last_error_string'}


def test_version_and_error_text(lib):
    assert lib.tkq_version() >= 100
    assert isinstance(lib.tkq_last_error_string(), bytes)


def test_argument_checks_need_no_device(lib):
    buf = (ctypes.c_char * 4096)()
    p = ctypes.addressof(buf)
    p16 = (p + 15) // 16 * 16
    # zero tokens: success, nothing launched
    assert lib.tkq_per_token_cast(p16, 0, 0, 256, 256, 0, 128, 0, p16, p16, 2, None) == 0
    # unknown dtype / format
    assert lib.tkq_per_token_cast(p16, 7, 4, 256, 256, 0, 128, 0, p16, p16, 2, None) == -1
    assert lib.tkq_per_token_cast(p16, 0, 4, 256, 256, 9, 128, 0, p16, p16, 2, None) == -1
    # null pointer
    assert lib.tkq_per_token_cast(None, 0, 4, 256, 256, 0, 128, 0, p16, p16, 2, None) == -1
    # unsupported group size, hidden not a multiple of 16, packed scales without the column-major flag
    assert lib.tkq_per_token_cast(p16, 0, 4, 256, 256, 0, 48, 0, p16, p16, 2, None) == -2
    assert lib.tkq_per_token_cast(p16, 0, 4, 248, 248, 0, 128, 0, p16, p16, 2, None) == -2
    assert lib.tkq_per_token_cast(p16, 0, 4, 256, 256, 0, 128, 4, p16, p16, 16, None) == -2
    assert b'column-major' in lib.tkq_last_error_string()
    # misaligned input
    assert lib.tkq_per_token_cast(p16 + 2, 0, 4, 256, 256, 0, 128, 0, p16, p16, 2, None) == -3
    # e5m6 needs one group per token; per-channel needs whole 128-token blocks
    assert lib.tkq_per_token_cast(p16, 0, 4, 256, 256, 2, 128, 0, p16, p16, 1, None) == -2
    assert lib.tkq_per_channel_cast(p16, 0, 100, 128, 0, p16, p16, None) == -2
    assert lib.tkq_per_block_cast(p16, 0, 4, 256, 0, 64, 64, 0, p16, p16, 2, None) == -2
    assert lib.tkq_swiglu_forward_and_per_token_cast(p16, 0, 4, 192, 128, None, None, None, -1.0, None, -1.0, 0, 0, p16, p16, 1,
                                                     None) == -2


def test_argument_checks_of_the_backward_and_expand_entry_points(lib):
    buf = (ctypes.c_char * 4096)()
    p16 = (ctypes.addressof(buf) + 15) // 16 * 16
    bwd = lib.tkq_swiglu_backward_and_per_token_cast
    # (x, x_sf, grad_out, weight, pos_to_token_topk, token_topk_to_pos, rows, hidden, tokens, topk, group, clamp, flags,
    #  out, x_grad_fp8, x_grad_sf, x_grad, weight_grad, stream)
    assert bwd(p16, p16, p16, p16, p16, p16, 0, 256, 2, 2, 128, -1.0, 0, p16, p16, p16, p16, p16, None) == 0       # no rows
    assert bwd(p16, p16, p16, p16, p16, p16, 4, 256, 2, 2, 64, -1.0, 0, p16, p16, p16, p16, p16, None) == -2      # group 64
    assert bwd(p16, p16, p16, p16, p16, p16, 4, 192, 2, 2, 128, -1.0, 0, p16, p16, p16, p16, p16, None) == -2     # 192 % 128
    assert bwd(p16, p16, p16, p16, p16, p16, 4, 256, 2, 2, 128, -1.0, 2, p16, p16, p16, p16, p16, None) == -2     # layout flag
    assert bwd(p16, None, p16, p16, p16, p16, 4, 256, 2, 2, 128, -1.0, 0, p16, p16, p16, p16, p16, None) == -1    # null
    assert bwd(p16 + 4, p16, p16, p16, p16, p16, 4, 256, 2, 2, 128, -1.0, 0, p16, p16, p16, p16, p16, None) == -3  # alignment
    expand = lib.tkq_expand_to_fused
    # (x, tokens, row_bytes, x_sf, sf_words, token_topk_to_pos, topk, pos_to_expert, expanded, flags, out, out_sf, stride, stream)
    assert expand(p16, 0, 256, None, 0, p16, 2, p16, 8, 0, p16, None, 0, None) == 0                                # no tokens
    assert expand(p16, 4, 250, None, 0, p16, 2, p16, 8, 0, p16, None, 0, None) == -2                               # 250 % 16
    assert expand(p16, 4, 256, p16, 0, p16, 2, p16, 8, 0, p16, p16, 2, None) == -1                                 # scales without a count
    assert expand(p16, 4, 256, None, 0, p16, 2, p16, 8, 4, p16, None, 0, None) == -2                               # unknown flag
    assert expand(p16 + 8, 4, 256, None, 0, p16, 2, p16, 8, 0, p16, None, 0, None) == -3                           # alignment
    assert b'expand_to_fused' in lib.tkq_last_error_string()


def test_argument_checks_of_the_quantized_input_entry_points(lib):
    buf = (ctypes.c_char * 4096)()
    p32 = (ctypes.addressof(buf) + 31) // 32 * 32
    lossless = lib.tkq_per_block_cast_lossless
    # (x, x_sf, x_sf_flags, x_sf_stride, x_block_m, x_block_k, tokens, hidden, x_row_stride, out_block_m, out_block_k, flags,
    #  out, sf, sf_stride, stream)
    assert lossless(p32, p32, 0, 8, 1, 32, 0, 256, 256, 128, 128, 0, p32, p32, 2, None) == 0          # no tokens
    assert lossless(p32, p32, 0, 8, 1, 32, 4, 256, 256, 64, 128, 0, p32, p32, 2, None) == -2         # output block 64 x 128
    assert lossless(p32, p32, 0, 8, 1, 32, 4, 240, 240, 128, 128, 0, p32, p32, 2, None) == -2        # hidden % 32
    assert lossless(p32, p32, 0, 8, 32, 32, 4, 256, 256, 1, 128, 0, p32, p32, 2, None) == -2         # output block below the input block
    assert lossless(p32, p32, 0, 8, 1, 32, 4, 256, 256, 128, 128, 4, p32, p32, 16, None) == -2       # packed scales, not column-major
    assert lossless(p32 + 8, p32, 0, 8, 1, 32, 4, 256, 256, 128, 128, 0, p32, p32, 2, None) == -3    # rows on 8-byte boundaries only
    assert lossless(p32, p32, 0, 8, 1, 32, 4, 256, 272, 128, 128, 0, p32, p32, 2, None) == -3        # row stride of 136 bytes
    assert b'per_block_cast_lossless' in lib.tkq_last_error_string()
    assert lossless(p32, None, 0, 8, 1, 32, 4, 256, 256, 128, 128, 0, p32, p32, 2, None) == -1       # null
    requant = lib.tkq_per_token_cast_quantized
    # (x, in_fmt, x_sf, x_sf_flags, x_sf_stride, x_block_m, x_block_k, tokens, hidden, x_row_stride, fmt, group, flags, out, sf,
    #  sf_stride, stream)
    assert requant(p32, 0, p32, 0, 2, 128, 128, 0, 256, 256, 0, 128, 0, p32, p32, 2, None) == 0      # no tokens
    assert requant(p32, 2, p32, 0, 2, 128, 128, 4, 256, 256, 0, 128, 0, p32, p32, 2, None) == -1     # E5M6 is not an input format
    assert requant(p32, 0, p32, 0, 2, 128, 128, 4, 256, 256, 0, 256, 0, p32, p32, 2, None) == -2     # one scale per token
    assert requant(p32, 0, p32, 4, 2, 128, 128, 4, 256, 256, 0, 128, 0, p32, p32, 2, None) == -2     # packed input scales, not column-major
    back = lib.tkq_cast_back
    # (x, in_fmt, x_sf, x_sf_flags, x_sf_stride, x_block_m, x_block_k, tokens, hidden, out_dtype, out, stream)
    assert back(p32, 0, p32, 0, 2, 1, 128, 0, 256, 0, p32, None) == 0                                 # no tokens
    assert back(p32, 0, p32, 0, 2, 1, 128, 4, 250, 0, p32, None) == -2                                # hidden % 16
    assert back(p32, 0, p32, 0, 2, 1, 128, 4, 256, 5, p32, None) == -1                                # output type
    assert back(p32 + 4, 0, p32, 0, 2, 1, 128, 4, 256, 0, p32, None) == -3                            # alignment


@pytest.mark.gpu
def test_bounded_wait_gives_up_and_reports(oracle, cuda_device):
    """The waits on asynchronous copies are bounded.  The self-test kernel receives one real copy, then waits a few
    thousand polls on a barrier nothing arrives on: it must return (nothing in flight, nothing faults), the device
    condition must read TKQ_DEVICE_WAIT_TIMEOUT once and then clear, and the next ordinary cast must be exact."""
    import torch
    from helpers import to_host
    from tilekernels_b200 import _lib, quant
    from tilekernels_b200.testing import assert_equal
    lib = _lib.lib()
    assert lib.tkq_device_error() == 0
    src = torch.arange(4, dtype=torch.int32, device=cuda_device) + 1234
    echo = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    stream = torch.cuda.current_stream(cuda_device).cuda_stream
    assert lib.tkq_selftest_bounded_wait(src.data_ptr(), 4096, echo.data_ptr(), stream) == 0
    torch.cuda.synchronize()
    assert int(echo.item()) == 1234          # the real copy arrived before the wait that runs out
    assert lib.tkq_device_error() == 1       # TKQ_DEVICE_WAIT_TIMEOUT
    assert lib.tkq_device_error() == 0
    assert lib.tkq_selftest_bounded_wait(src.data_ptr(), 0, None, stream) == -1   # limit out of range: nothing launched
    x = torch.randn((256, 512), generator=torch.Generator().manual_seed(1)).to(torch.bfloat16)
    out, sf = quant.per_block_cast(x.to(cuda_device), 'e4m3', (128, 128))
    want = oracle.cast(x, 'e4m3', (128, 128))
    assert_equal(to_host(out), want[0])
    assert_equal(to_host(sf), want[1])
    assert lib.tkq_device_error() == 0
